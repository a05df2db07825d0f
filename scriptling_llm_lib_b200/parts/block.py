"""How a layer's parts are arranged around the residual stream.

A layer is data: the name of an arrangement and the parts it is made of, by role. An arrangement
(a block class) builds its parts from their registries, runs them in its order, and answers for
the layer: which parts it has, whether its decode step can be captured, what it needs of the cache.
The engine asks the block, never a part by name, so an arrangement with other roles (no
feed-forward, two mixers, four norms) is a class of its own and nothing else changes.

"pre_norm": x += mixer(norm(x)); x += feed_forward(norm(x)) (model_f32.go:382-500), roles
`mixer_norm`, `mixer`, `feed_forward_norm`, `feed_forward`. The residual stream is float32; a block
hands its last sublayer's output on as a pending `delta`, which the next norm adds while it reads
the row, so no separate pass over the stream is needed.

Where the norm between two sublayers and the products on either side of it all agree (see base.py:
FoldRequest, Folded), the norm needs no kernel: the block asks the sublayer before it to finish the
residual sum and prepare the norm's output, and hands the result through the norm to the sublayer
behind it. Across layers the same holds for a layer's first norm: a block that sets `folds_entry`
tells through `entry_fold(ctx, rows, residual)` what the layer before it may prepare, and accepts
that layer's request as `forward(..., next_fold=...)`.

A block's interface:
  parts() -> list of its parts                  for tensor specs, bind, prepare
  forward(residual, delta, ctx, unit, writes) -> delta
  graph_safe() -> bool                          its decode step launches the same work whatever the values
  cache_need() -> CacheNeed | None              what the cache unit it writes must hold
  state_need() -> StateNeed | None              per-sequence state of fixed size
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Mapping

from .base import ARRANGEMENTS, FEED_FORWARDS, MIXERS, NORMS, STREAM_INPUTS, FoldRequest, PartSpec


@dataclass(frozen=True)
class LayerSpec:
    """One layer as data: the arrangement, its parts by role, and the arrangement's own constants."""
    arrangement: str
    parts: Mapping[str, PartSpec] = field(default_factory=dict)
    params: Mapping[str, object] = field(default_factory=dict)


def pre_norm_layer(mixer: PartSpec, feed_forward: PartSpec, mixer_norm: PartSpec, feed_forward_norm: PartSpec) -> LayerSpec:
    return LayerSpec("pre_norm", dict(mixer=mixer, feed_forward=feed_forward, mixer_norm=mixer_norm,
                                      feed_forward_norm=feed_forward_norm))


import os
_NO_FOLD = bool(os.environ.get("SLLM_NO_FOLD"))


def fold_request(norm, before, behind, ctx, rows: int, residual):
    """A FoldRequest for `norm` if it, the part `before` it and the part `behind` it all can; else None.
    What the three answer depends on a step only through its kind (how many rows, decode or not), so
    the answer is kept per kind, with the norm (which lives and dies with its neighbours)."""
    if _NO_FOLD:
        return None
    memo = norm.__dict__.setdefault("_fold_memo", {})
    key = (id(before), id(behind), min(rows, 256), bool(ctx.is_decode), ctx.dtype)
    try:
        terms = memo[key]
    except KeyError:
        terms = norm.fold_terms() if hasattr(norm, "fold_terms") else None
        can = getattr(before, "can_fold", None)
        takes = getattr(behind, "takes_folded", None)
        if terms is None or can is None or takes is None or not can(ctx, rows) or not takes(ctx, rows):
            terms = None
        memo[key] = terms
    return None if terms is None else FoldRequest(residual, terms[0], terms[1])


class Block:
    """Base of the arrangements: answers for the layer out of `parts()`; an arrangement with one
    mixer need only name it `self.mixer`."""
    mixer = None
    folds_entry = False          # True: forward takes next_fold=..., and entry_fold says what may be prepared for it

    def parts(self) -> list:
        raise NotImplementedError

    def forward(self, residual, delta, ctx, unit, writes):
        raise NotImplementedError

    def graph_safe(self) -> bool:
        return all(getattr(p, "graph_safe", False) for p in self.parts())

    def cache_need(self):
        return self.mixer.cache_need() if self.mixer is not None else None

    def state_need(self):
        return self.mixer.state_need() if self.mixer is not None else None


def _role(spec: LayerSpec, role: str) -> PartSpec:
    try:
        return spec.parts[role]
    except KeyError:
        raise ValueError(f"the {spec.arrangement!r} arrangement needs a part in the role {role!r}; "
                         f"the layer has {', '.join(sorted(spec.parts)) or 'none'}") from None


class PreNormBlock(Block):
    def __init__(self, spec: LayerSpec):
        self.mixer_norm = NORMS.build(_role(spec, "mixer_norm"))
        self.mixer = MIXERS.build(_role(spec, "mixer"))
        self.feed_forward_norm = NORMS.build(_role(spec, "feed_forward_norm"))
        self.feed_forward = FEED_FORWARDS.build(_role(spec, "feed_forward"))

    def parts(self):
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    folds_entry = True

    def entry_fold(self, ctx, rows: int, residual, before):
        """What the sublayer `before` this layer may prepare of this layer's first norm (or None)."""
        return fold_request(self.mixer_norm, before, self.mixer, ctx, rows, residual)

    def last_part(self):
        return self.feed_forward

    def forward(self, residual, delta, ctx, unit, writes, next_fold=None):
        """residual float32 [T, hidden] (updated in place), delta: pending addend or None (or the
        prepared output of this layer's first norm). Returns the new pending addend; `next_fold`
        (a function of the part that would do it) asks the last sublayer to prepare the next
        layer's first norm instead."""
        rows = residual.shape[0]
        n = self.mixer_norm.forward(residual, delta, ctx)
        fold = fold_request(self.feed_forward_norm, self.mixer, self.feed_forward, ctx, rows, residual)
        a = self.mixer.forward(n, ctx, unit, writes, fold=fold) if fold is not None else self.mixer.forward(n, ctx, unit, writes)
        n2 = self.feed_forward_norm.forward(residual, a, ctx)
        fold = next_fold(self.feed_forward) if next_fold is not None else None
        return self.feed_forward.forward(n2, ctx, fold=fold) if fold is not None else self.feed_forward.forward(n2, ctx)


class ScaledPreNormBlock(Block):
    """x += m * mixer(c(norm(x))); then, if the layer has a feed-forward, x += m * feed_forward(norm(x)).

    m (`residual_scale`) multiplies every sublayer's output on its way into the residual stream.
    c (`input_conv`, optional) is a short causal convolution over time on each channel of what the
    mixer reads, with the input added back: c(h) = h + conv(h); its last taps - 1 inputs are state
    of the sequence like a recurrent mixer's. Roles: `mixer_norm`, `mixer`, and either both or
    neither of `feed_forward_norm`, `feed_forward`. A sublayer's output goes on as weighted addends
    (tensor, coefficient), so the norms named here must take those (`weighted_norm`); a mixer may
    return such a list itself (branches side by side), and m multiplies its coefficients. The
    unit's state is {"input_conv": ..., "mixer": ...} with whichever of the two exist."""

    def __init__(self, spec: LayerSpec):
        from .conv import CausalConv
        self.mixer_norm = NORMS.build(_role(spec, "mixer_norm"))
        self.mixer = MIXERS.build(_role(spec, "mixer"))
        has = [r in spec.parts for r in ("feed_forward_norm", "feed_forward")]
        if has[0] != has[1]:
            raise ValueError("a layer has a feed-forward and its norm, or neither")
        self.feed_forward_norm = NORMS.build(spec.parts["feed_forward_norm"]) if has[0] else None
        self.feed_forward = FEED_FORWARDS.build(spec.parts["feed_forward"]) if has[1] else None
        self.scale = float(spec.params.get("residual_scale", 1.0))
        conv = spec.params.get("input_conv")
        self.input_conv = CausalConv([conv["name"]], [int(conv["channels"])], int(conv["taps"]), residual=True) if conv else None

    def parts(self):
        out = [self.mixer_norm, self.mixer]
        if self.input_conv is not None:
            out.append(self.input_conv)
        if self.feed_forward is not None:
            out += [self.feed_forward_norm, self.feed_forward]
        return out

    def graph_safe(self) -> bool:
        return all(getattr(p, "graph_safe", False) for p in self.parts() if p is not self.input_conv)

    def state_need(self):
        need = {}
        if self.input_conv is not None and self.input_conv.state_need() is not None:
            need["input_conv"] = self.input_conv.state_need()
        if self.mixer.state_need() is not None:
            need["mixer"] = self.mixer.state_need()
        return need or None

    def _scaled(self, y):
        """A sublayer's output as addends with the residual scale applied."""
        import torch
        if isinstance(y, torch.Tensor):
            return [(y[i], self.scale) for i in range(y.shape[0])] if y.dim() == 3 else [(y, self.scale)]
        return [(t, c * self.scale) for t, c in y]

    def forward(self, residual, delta, ctx, unit, writes):
        st = ctx.unit_state(unit) if self.state_need() is not None else {}
        h = self.mixer_norm.forward(residual, delta, ctx)
        if self.input_conv is not None:
            h = self.input_conv.forward(h, st.get("input_conv"), ctx, ctx.dtype)
        if "mixer" in st:
            a = self.mixer.forward(h, ctx, unit, writes, state=st["mixer"])
        else:
            a = self.mixer.forward(h, ctx, unit, writes)
        a = self._scaled(a)
        if self.feed_forward is None:
            return a
        n2 = self.feed_forward_norm.forward(residual, a, ctx)
        return self._scaled(self.feed_forward.forward(n2, ctx))


class SandwichNormBlock(Block):
    """x += post1(mixer(pre1(x))); then, if the layer has a feed-forward, x += post2(feed_forward(pre2(x))):
    a norm in front of and behind every sublayer. Roles: `mixer_norm`, `mixer`, `mixer_post_norm`, and
    all or none of `feed_forward_norm`, `feed_forward`, `feed_forward_post_norm`. The norm behind a
    sublayer does not run by itself: the sublayer's output goes on as a `NormedAddend`, and the norm
    that reads the stream next (this layer's second, the next layer's first, or the model's last)
    applies it while it adds, so the norms named here must take such addends (`dynamic_tanh`)."""

    def __init__(self, spec: LayerSpec):
        self.mixer_norm = NORMS.build(_role(spec, "mixer_norm"))
        self.mixer = MIXERS.build(_role(spec, "mixer"))
        self.mixer_post_norm = NORMS.build(_role(spec, "mixer_post_norm"))
        roles = ("feed_forward_norm", "feed_forward", "feed_forward_post_norm")
        has = [r in spec.parts for r in roles]
        if any(has) and not all(has):
            raise ValueError("a layer has a feed-forward with a norm on either side, or none of the three")
        self.feed_forward_norm = NORMS.build(spec.parts[roles[0]]) if has[0] else None
        self.feed_forward = FEED_FORWARDS.build(spec.parts[roles[1]]) if has[1] else None
        self.feed_forward_post_norm = NORMS.build(spec.parts[roles[2]]) if has[2] else None

    def parts(self):
        out = [self.mixer_norm, self.mixer, self.mixer_post_norm]
        if self.feed_forward is not None:
            out += [self.feed_forward_norm, self.feed_forward, self.feed_forward_post_norm]
        return out

    def forward(self, residual, delta, ctx, unit, writes):
        from .norm import NormedAddend
        h = self.mixer_norm.forward(residual, delta, ctx)
        pending = NormedAddend(self.mixer.forward(h, ctx, unit, writes), self.mixer_post_norm)
        if self.feed_forward is None:
            return pending
        h2 = self.feed_forward_norm.forward(residual, pending, ctx)
        return NormedAddend(self.feed_forward.forward(h2, ctx), self.feed_forward_post_norm)


class PreNormInputBlock(Block):
    """x += mixer(norm(x)); then, where the layer has a feed-forward, x += feed_forward(norm(x)); then, where it has
    one, a stream input: a part that reads the stream as it stands and the step's tokens and adds to it. Roles:
    `mixer_norm`, `mixer`, both or neither of `feed_forward_norm`, `feed_forward`, and optionally `stream_input`.
    The mixer may keep per-sequence state (it is handed the unit's as `state=`); the norms are of the kind that
    takes a plain pending addend or one that is still to be divided by its own root mean square (`rmsnorm`)."""

    def __init__(self, spec: LayerSpec):
        self.mixer_norm = NORMS.build(_role(spec, "mixer_norm"))
        self.mixer = MIXERS.build(_role(spec, "mixer"))
        has = [r in spec.parts for r in ("feed_forward_norm", "feed_forward")]
        if has[0] != has[1]:
            raise ValueError("a layer has a feed-forward and its norm, or neither")
        self.feed_forward_norm = NORMS.build(spec.parts["feed_forward_norm"]) if has[0] else None
        self.feed_forward = FEED_FORWARDS.build(spec.parts["feed_forward"]) if has[1] else None
        self.stream_input = STREAM_INPUTS.build(spec.parts["stream_input"]) if "stream_input" in spec.parts else None

    def parts(self):
        out = [self.mixer_norm, self.mixer]
        if self.feed_forward is not None:
            out += [self.feed_forward_norm, self.feed_forward]
        if self.stream_input is not None:
            out.append(self.stream_input)
        return out

    @staticmethod
    def _addend(y, ctx):
        """A sublayer's output in a form the norms take: float32 sums of a 16-bit engine travel as one partial sum."""
        import torch
        if isinstance(y, torch.Tensor) and y.dim() == 2 and y.dtype == torch.float32 and ctx.dtype != torch.float32:
            return y.unsqueeze(0)
        return y

    def forward(self, residual, delta, ctx, unit, writes):
        st = ctx.unit_state(unit) if self.state_need() is not None else None
        h = self.mixer_norm.forward(residual, delta, ctx)
        a = self.mixer.forward(h, ctx, unit, writes, state=st) if st is not None else self.mixer.forward(h, ctx, unit, writes)
        a = self._addend(a, ctx)
        if self.feed_forward is not None:
            h2 = self.feed_forward_norm.forward(residual, a, ctx)
            a = self._addend(self.feed_forward.forward(h2, ctx), ctx)
        if self.stream_input is None:
            return a
        return self.stream_input.forward(residual, a, ctx)


class ParallelInputBlock(Block):
    """x += mixer(h) + feed_forward(h) with h = norm(x): ONE norm, and both sublayers read its output; then, where the layer
    has one, a stream input (a part that reads the stream as it then stands and the step's tokens and adds to it). Roles:
    `mixer_norm`, `mixer`, optionally `feed_forward`, optionally `stream_input`. The sublayers' outputs travel as a list of
    addends (a feed-forward may itself answer with a list: routed experts beside an expert that every token uses), taken
    into the stream in one pass by the stream input or by the norm that reads the stream next, so the norms named here must
    take lists (`dynamic_tanh`). The mixer may keep per-sequence state (handed to it as `state=`)."""

    def __init__(self, spec: LayerSpec):
        self.mixer_norm = NORMS.build(_role(spec, "mixer_norm"))
        self.mixer = MIXERS.build(_role(spec, "mixer"))
        self.feed_forward = FEED_FORWARDS.build(spec.parts["feed_forward"]) if "feed_forward" in spec.parts else None
        self.stream_input = STREAM_INPUTS.build(spec.parts["stream_input"]) if "stream_input" in spec.parts else None

    def parts(self):
        out = [self.mixer_norm, self.mixer]
        if self.feed_forward is not None:
            out.append(self.feed_forward)
        if self.stream_input is not None:
            out.append(self.stream_input)
        return out

    def forward(self, residual, delta, ctx, unit, writes):
        st = ctx.unit_state(unit) if self.state_need() is not None else None
        h = self.mixer_norm.forward(residual, delta, ctx)
        a = self.mixer.forward(h, ctx, unit, writes, state=st) if st is not None else self.mixer.forward(h, ctx, unit, writes)
        pending = list(a) if isinstance(a, (list, tuple)) else [a]
        if self.feed_forward is not None:
            f = self.feed_forward.forward(h, ctx)
            pending += list(f) if isinstance(f, (list, tuple)) else [f]
        if self.stream_input is None:
            return pending
        return self.stream_input.forward(residual, pending, ctx)


ARRANGEMENTS.register("pre_norm", PreNormBlock)
ARRANGEMENTS.register("parallel_input", ParallelInputBlock)
ARRANGEMENTS.register("pre_norm_input", PreNormInputBlock)
ARRANGEMENTS.register("sandwich_norm", SandwichNormBlock)
ARRANGEMENTS.register("scaled_pre_norm", ScaledPreNormBlock)


def build_block(spec: LayerSpec):
    return ARRANGEMENTS.build(PartSpec(spec.arrangement), spec=spec)

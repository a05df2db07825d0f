"""Grouped-query causal attention over the paged cache.

q = x Wq^T, k = x Wk^T, v = x Wv^T; Q and K rotated by the position encoding; K, V appended to
the cache; query head h reads key/value head h // (H/G); score = (q.k) / sqrt(head_dim); keys
after the query are masked; max-subtracted softmax; out = sum p v; y = out Wo^T
(model_f32.go:391-470, float32_ops.go:190-235, :252-260). A `window` (absent in the reference)
also masks keys `window` or more positions behind the query and lets the cache give old pages
back. With `writes=False` the layer projects queries only and reads the unit another layer wrote.
Two more options, both absent in the reference: value heads of a width of their own (`v_dim`; the
cache then keeps values that wide and the output product reads n_heads * v_dim columns), and
`value_norm_eps`: every value head is divided by its root mean square, sqrt(mean(v^2) + eps),
before it is cached. Either sends the step's keys and values through a store kernel that does
rotation, value norm and cache write in one pass (`kv_store`); values as wide as keys then still
use the attention kernels below, other widths a kernel that takes both (`attn_wide_value`).

Four more options, none in the reference. `chunk`: a query sees the earlier keys of its own chunk of that many
positions only, chunks counted from position 0 of the sequence (not from where a step begins); the cache
gives pages back once the chunk they belong to has passed. `conv`: a short causal convolution over time on
every channel of the projected queries, keys and values, straight behind the projection; the last taps - 1
projected rows of a sequence are its state. `qk_norm`: queries and keys are each divided by the root mean
square of the WHOLE projection (all heads at once) and multiplied by a weight of that size, before the
rotation. `gate_name`: a matrix [n_heads, hidden] on the mixer's own input; head h's output is multiplied by
the sigmoid of its logit before the output product. With `conv` or `qk_norm` the step's rows go through one
kernel that norms, rotates and fills the cache in float32: `conv_qk_norm_store` does the convolution too and
keeps its float32 output on the chip (rows up to 51200 columns); `qk_norm_store` reads the float32 output of a
convolution that ran by itself, or the projection. The attention kernels are the same ones.

Four more, again none in the reference. `values_are_keys`: there is no value projection; a position's values are its keys
as projected, before the rotation (the cache keeps both: the turned keys and the unturned ones as values; the key
matrix is stacked twice into the one product, so every kernel behind it sees the usual q|k|v row). `softcap`: a score
s = (q . k) * scale becomes softcap * tanh(s / softcap) before the softmax. `sink_name`: a stored logit per head
that takes part in the softmax's normalisation only: exp(sink) is added to the denominator once, however many keys there
are and however a step splits them; nothing goes to the numerator, and neither the scale nor the cap touches it. `gate_per="element"`: the gate matrix is [n_heads * v_dim, hidden] and the
concatenated heads are multiplied element by element with the sigmoid of its product with the mixer's input
("head", the default: one logit per head). Capped scores and sinks are known to the attention kernels of the generic set
(both precisions; scores, cap, softmax and sink float32) and, in bfloat16 with heads of 64 or 128, to the tcgen05 prompt
kernels and to the decode kernel that puts a group's query heads on the tensor cores.

The position encoding is optional (`position=None`: queries and keys as projected). Storing keys
and values in the cache is this mixer's own step, whatever the encoding: for an encoding that is a
rotation by a table the store and the rotation are one kernel (or part of the q|k|v product's
epilogue, or of the decode attention kernel, where the widths allow); any other encoding rewrites
the step's query and key rows in place first (`transform`) and the store copies.
"""
from __future__ import annotations

import math

import torch

from ..cache.needs import CacheNeed
from ..csrc.bindings import DecodeKernels, PrefillAttentionTC
from ..cache.needs import StateNeed
from ..weights.spec import TensorSpec
from .base import MIXERS, POSITION_ENCODINGS, Folded, Mixer, PartSpec
from .conv import CausalConv
from .linear import Linear


class Attention(Mixer):
    @property
    def graph_safe(self) -> bool:
        """The decode step launches the same work whatever the values; an encoding that rewrites rows
        itself (`transform`) has to say the same of its own work."""
        return self.position is None or self.position.rotation() is not None or bool(getattr(self.position, "graph_safe", False))

    def __init__(self, hidden: int, n_heads: int, n_kv_heads: int, head_dim: int, position: PartSpec | None,
                 q_name: str, k_name: str, v_name: str, o_name: str, window: int | None = None,
                 scale: float | None = None, v_dim: int | None = None, value_norm_eps: float | None = None,
                 chunk: int | None = None, conv: dict | None = None, qk_norm: dict | None = None, gate_name: str | None = None,
                 values_are_keys: bool = False, softcap: float | None = None, sink_name: str | None = None,
                 gate_per: str = "head"):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads cannot share {n_kv_heads} key/value heads")
        if not 1 <= head_dim <= 512:
            raise ValueError(f"head_dim {head_dim}: the attention kernels take head widths 1..512")
        if window and chunk:
            raise ValueError("an attention layer has a sliding window or chunks, not both")
        if chunk is not None and chunk < 1:
            raise ValueError(f"chunks of {chunk} positions")
        if gate_per not in ("head", "element"):
            raise ValueError(f"a gate per {gate_per!r}; known: head, element")
        self.values_are_keys = bool(values_are_keys)
        if self.values_are_keys:
            if v_dim is not None and int(v_dim) != head_dim:
                raise ValueError(f"values that are the keys are as wide as the keys ({head_dim}), not {v_dim}")
            if conv is not None or value_norm_eps is not None:
                raise ValueError("values that are the keys take neither a convolution nor a value norm")
            v_name = k_name
        self.softcap = float(softcap) if softcap else None
        if self.softcap is not None and not self.softcap > 0:
            raise ValueError(f"a cap on the scores must be positive, got {softcap}")
        self.sink_name, self.sink = sink_name, None
        self.plain_softmax = self.softcap is None and sink_name is None
        if not self.plain_softmax and v_dim is not None and int(v_dim) != head_dim:
            raise ValueError("capped scores and sinks run on kernels whose values are as wide as the keys")
        self.gate_per = gate_per
        self.hidden, self.n_heads, self.n_kv_heads, self.head_dim, self.window = hidden, n_heads, n_kv_heads, head_dim, window
        self.chunk = int(chunk) if chunk else None
        # what the kernels take as `window`: > 0 a sliding window, < 0 chunks of that many positions, 0 every earlier key
        self.span = int(window) if window else (-self.chunk if self.chunk else 0)
        self.v_dim = head_dim if v_dim is None else int(v_dim)
        self.value_norm_eps = None if value_norm_eps is None else float(value_norm_eps)
        if self.v_dim < 1 or self.v_dim > 512:
            raise ValueError(f"value heads of width {self.v_dim}: the attention kernels take 1..512")
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.position = POSITION_ENCODINGS.build(position) if position is not None else None
        qw, kw = n_heads * head_dim, n_kv_heads * head_dim
        vw = n_kv_heads * self.v_dim
        self.gate_name = gate_name
        names, widths = [q_name, k_name, v_name], [qw, kw, vw]
        if gate_name is not None:               # the gates' logits ride in the same product, behind the values
            names, widths = names + [gate_name], widths + [n_heads if gate_per == "head" else n_heads * self.v_dim]
        self.qkv = Linear(names, widths, hidden)
        self.out = Linear([o_name], [hidden], n_heads * self.v_dim)
        self.q_only: Linear | None = None
        self.conv = None
        if conv is not None and int(conv["taps"]) > 1:
            self.conv = CausalConv([conv["q_name"], conv["k_name"], conv["v_name"]], [qw, kw, vw], int(conv["taps"]))
        self.qk_norm = dict(qk_norm) if qk_norm is not None else None
        self.q_norm_w = self.k_norm_w = None

    @property
    def prepared(self) -> bool:
        """The step's rows pass the convolution and / or the whole-projection norm on their way into the cache."""
        return self.conv is not None or self.qk_norm is not None

    def tensor_specs(self):
        specs, seen = [], set()
        for ts in self.qkv.tensor_specs() + self.out.tensor_specs():      # the key matrix may stand twice in the stacked product
            if ts.name not in seen:
                seen.add(ts.name)
                specs.append(ts)
        if self.sink_name is not None:
            specs.append(TensorSpec(self.sink_name, (self.n_heads,), init="bias"))
        if self.conv is not None:
            specs += self.conv.tensor_specs()
        if self.qk_norm is not None:
            specs += [TensorSpec(self.qk_norm["q_name"], (self.n_heads * self.head_dim,), init="norm_weight"),
                      TensorSpec(self.qk_norm["k_name"], (self.n_kv_heads * self.head_dim,), init="norm_weight")]
        return specs

    def bind(self, tensors, dtype, device):
        self.qkv.bind(tensors, dtype, device)
        self.out.bind(tensors, dtype, device)
        self.q_only = self.qkv.rows(0, self.n_heads * self.head_dim)
        if self.sink_name is not None:
            self.sink = tensors[self.sink_name].float().contiguous()
        if self.conv is not None:
            self.conv.bind(tensors, dtype, device)
        if self.qk_norm is not None:
            self.q_norm_w = tensors[self.qk_norm["q_name"]].float().contiguous()
            self.k_norm_w = tensors[self.qk_norm["k_name"]].float().contiguous()

    def state_need(self):
        need = self.conv.state_need() if self.conv is not None else None
        return {"conv": need} if need is not None else None

    def prepare(self, max_positions, device):
        if self.position is not None:
            self.position.prepare(max_positions, device)

    def _store(self, qkv, ctx, rotation, n_kv, kpages, vpages, block_table) -> None:
        """Give the step's queries and keys their positions and append keys and values to the cache
        (n_kv == 0: queries only). `rotation`: the encoding's table, or None."""
        if self.position is not None and rotation is None:
            self.position.transform(qkv, ctx, self.n_heads, n_kv, self.head_dim)
        if rotation is None and n_kv == 0:
            return
        table, rot, interleaved = rotation if rotation is not None else (None, 0, False)
        if self.own_store:
            ctx.kernels.seq.kv_store(qkv, ctx.tok_pos, ctx.tok_seq, block_table, table, kpages, vpages, self.n_heads, n_kv,
                                     self.head_dim, self.v_dim, rot, interleaved, self.value_norm_eps)
            return
        ctx.kernels.rope_kv_write(qkv, ctx.tok_pos, ctx.tok_seq, block_table, table, kpages, vpages, self.n_heads, n_kv,
                                  self.head_dim, rot, interleaved)

    def cache_need(self):
        kind = "window" if self.window else "chunk" if self.chunk else "full"
        return CacheNeed(kind, self.n_kv_heads, self.head_dim, self.window or self.chunk,
                         v_dim=None if self.v_dim == self.head_dim else self.v_dim)

    @property
    def own_store(self) -> bool:
        """Keys and values go through `kv_store` (value norm, or values of another width than keys)."""
        return self.value_norm_eps is not None or self.other_widths

    @property
    def other_widths(self) -> bool:
        """Values of another width than keys, or a head width off the steps of 16 that the tiled and
        tensor-core attention kernels are built for: `attn_wide_value` takes any."""
        return self.v_dim != self.head_dim or self.head_dim % 16 != 0

    def takes_folded(self, ctx, rows: int) -> bool:
        """The q|k|v product can scale its own output rows: in a decode step of few rows, and in a long
        prompt step (the tensor-core product, with or without the rotation in its epilogue)."""
        if self.prepared or self.gate_name is not None or not self.plain_softmax:
            return False
        path = self.qkv.fold_path(ctx, rows, ctx.dtype)
        return path is not None and self.q_only.fold_path(ctx, rows, ctx.dtype) == path and (ctx.is_decode or path == "tiles")

    def can_fold(self, ctx, rows: int) -> bool:
        """The output product can finish the sublayer: add to the residual stream and prepare the next norm."""
        path = self.out.fold_path(ctx, rows, ctx.dtype, finishing=True)
        return path is not None and (ctx.is_decode or path == "tiles")

    def _attend(self, qkv, x, ctx, kpages, vpages, block_table, fast_decode, fusion, writes):
        """The step's queries (the leading columns of `qkv`) over the cache -> [T, n_heads * v_dim]."""
        attn = torch.empty((x.shape[0], self.n_heads * self.v_dim), dtype=x.dtype, device=x.device)
        if not self.plain_softmax:
            k = ctx.kernels
            if not qkv.is_contiguous():
                qkv = qkv.contiguous()
            dec = ctx.kernels.decode if x.dtype == torch.bfloat16 else None
            if (ctx.is_decode and dec is not None and self.head_dim in (64, 128)
                    and dec.uses_tensor_cores(ctx.n_seqs, self.n_heads, self.n_kv_heads, self.head_dim)):
                # the decode kernel that puts a group's query heads on the tensor cores knows the cap and the sink
                n_split = ctx.decode_splits(self.n_heads, self.n_kv_heads, self.head_dim)
                scratch = torch.empty((ctx.n_seqs * self.n_heads * n_split * (self.head_dim + 2),), dtype=torch.float32,
                                      device=x.device)
                dec.attn_decode_capped(qkv, attn, ctx.seq_pos0, block_table, kpages, vpages, scratch,
                                       ctx.engine.tickets(ctx.n_seqs * self.n_kv_heads), ctx.n_seqs, self.n_heads, self.n_kv_heads,
                                       self.head_dim, self.span, self.scale, n_split, self.softcap, self.sink)
            elif not ctx.is_decode and x.dtype == torch.bfloat16 and self.head_dim in PrefillAttentionTC.HEAD_DIMS:
                ctx.kernels.prefill_attention_tc.attn(qkv, attn, ctx.seq_start, ctx.seq_pos0, block_table, kpages, vpages,
                                                      ctx.n_seqs, ctx.max_new, self.n_heads, self.n_kv_heads, self.head_dim,
                                                      self.span, self.scale, ctx.err_flag, self.softcap, self.sink)
            elif ctx.is_decode and k.attn_decode_split_takes(self.head_dim, qkv.stride(0)):
                n_split = k.attn_decode_splits(ctx.n_seqs, self.n_heads, self.n_kv_heads, ctx.max_pages, ctx.engine.sm_count)
                part = torch.empty((ctx.n_seqs * self.n_heads * n_split * (self.head_dim + 2),), dtype=torch.float32,
                                   device=x.device) if n_split > 1 else None
                k.attn_decode_split(qkv, attn, ctx.seq_pos0, block_table, kpages, vpages, part, ctx.n_seqs, self.n_heads,
                                    self.n_kv_heads, self.head_dim, self.span, self.scale, n_split, self.softcap, self.sink)
            else:
                k.attn_paged(qkv, attn, ctx.seq_start, ctx.seq_pos0, block_table, kpages, vpages, ctx.n_seqs, ctx.max_new,
                             self.n_heads, self.n_kv_heads, self.head_dim, self.span, self.scale, self.softcap, self.sink)
        elif self.other_widths:
            ctx.kernels.seq.attn_wide_value(qkv, attn, ctx.tok_pos, ctx.tok_seq, block_table, kpages, vpages, self.n_heads,
                                            self.n_kv_heads, self.head_dim, self.v_dim, self.span, self.scale)
        elif fast_decode:
            n_split = ctx.decode_splits(self.n_heads, self.n_kv_heads, self.head_dim)
            scratch = torch.empty((ctx.n_seqs * self.n_heads * n_split * (self.head_dim + 2),), dtype=torch.float32,
                                  device=x.device)
            tickets = ctx.engine.tickets(ctx.n_seqs * self.n_kv_heads)
            if fusion is not None:      # rotation and cache write happen inside the attention kernel
                ctx.kernels.decode.attn_decode_rope(qkv, attn, ctx.seq_pos0, block_table, kpages, vpages, scratch, tickets,
                                                    fusion[0], fusion[1], fusion[2], writes, ctx.n_seqs, self.n_heads,
                                                    self.n_kv_heads, self.head_dim, self.span, self.scale, n_split)
            else:
                ctx.kernels.decode.attn_decode(qkv, attn, ctx.seq_pos0, block_table, kpages, vpages, scratch, ctx.n_seqs,
                                               self.n_heads, self.n_kv_heads, self.head_dim, self.span, self.scale,
                                               n_split, tickets=tickets)
        elif x.dtype == torch.bfloat16 and self.head_dim in PrefillAttentionTC.HEAD_DIMS:
            ctx.kernels.prefill_attention_tc.attn(qkv, attn, ctx.seq_start, ctx.seq_pos0, block_table, kpages, vpages,
                                                  ctx.n_seqs, ctx.max_new, self.n_heads, self.n_kv_heads, self.head_dim,
                                                  self.span, self.scale, ctx.err_flag)
        elif ctx.is_decode and ctx.kernels.attn_decode_split_takes(self.head_dim, qkv.stride(0)):
            # one query per sequence on the generic path (the whole 32-bit decode step): keys split over blocks
            n_split = ctx.kernels.attn_decode_splits(ctx.n_seqs, self.n_heads, self.n_kv_heads, ctx.max_pages, ctx.engine.sm_count)
            part = torch.empty((ctx.n_seqs * self.n_heads * n_split * (self.head_dim + 2),), dtype=torch.float32,
                               device=x.device) if n_split > 1 else None
            ctx.kernels.attn_decode_split(qkv, attn, ctx.seq_pos0, block_table, kpages, vpages, part, ctx.n_seqs,
                                          self.n_heads, self.n_kv_heads, self.head_dim, self.span, self.scale, n_split)
        else:
            ctx.kernels.attn_paged(qkv, attn, ctx.seq_start, ctx.seq_pos0, block_table, kpages, vpages, ctx.n_seqs,
                                   ctx.max_new, self.n_heads, self.n_kv_heads, self.head_dim, self.span, self.scale)
        return attn

    def _forward_prepared(self, x, ctx, writes, state, kpages, vpages, block_table, fold):
        """The path of a layer with a convolution, a whole-projection norm or a gate: one product for queries, keys,
        values and gate logits; convolution (float32 out); norm, rotation and cache write in one kernel; attention;
        gate; output product."""
        if not writes:
            raise ValueError("a layer with a convolution, a query/key norm or a gate fills its own cache unit")
        T = x.shape[0]
        qw, kw, vw = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim, self.n_kv_heads * self.v_dim
        y = self.qkv.forward(x, ctx)
        c = y[:, :qw + kw + vw]
        k = ctx.kernels.gate
        fused_conv = (self.conv is not None and self.conv.plain and c.dtype == ctx.dtype
                      and qw + kw + vw <= k.FUSED_CONV_MAX_WIDTH)
        if self.conv is not None and not fused_conv:
            c = self.conv.forward(c, state["conv"], ctx, torch.float32)
        rotation = self.position.rotation() if self.position is not None else None
        if self.position is not None and rotation is None:
            raise ValueError("a layer with a convolution or a query/key norm takes a position encoding that is a rotation")
        table, rot, interleaved = rotation if rotation is not None else (None, 0, False)
        q = torch.empty((T, qw), dtype=x.dtype, device=x.device)
        eps = float(self.qk_norm["eps"]) if self.qk_norm is not None else 0.0
        if fused_conv:     # the convolution's output stays on the chip: one kernel from the projection to the cache
            k.conv_qk_norm_store(c, self.conv.weight, self.conv.taps, state["conv"], ctx, q, block_table, table, kpages, vpages,
                                 self.n_heads, self.n_kv_heads, self.head_dim, self.v_dim, rot, interleaved, self.q_norm_w,
                                 self.k_norm_w, eps)
        else:
            k.qk_norm_store(c, q, ctx.tok_pos, ctx.tok_seq, block_table, table, kpages, vpages, self.n_heads,
                            self.n_kv_heads, self.head_dim, self.v_dim, rot, interleaved, self.q_norm_w, self.k_norm_w, eps)
        fast_decode = (ctx.is_decode and x.dtype == torch.bfloat16 and self.head_dim in DecodeKernels.HEAD_DIMS
                       and not self.other_widths)
        attn = self._attend(q, x, ctx, kpages, vpages, block_table, fast_decode, None, writes)
        if self.gate_name is not None and self.gate_per == "head":
            ctx.kernels.gate.head_gate(attn, y[:, qw + kw + vw:], self.n_heads, self.v_dim)
        elif self.gate_name is not None:            # a logit per element: "heads" of one column each
            ctx.kernels.gate.head_gate(attn, y[:, qw + kw + vw:], self.n_heads * self.v_dim, 1)
        if fold is not None:
            return self.out.forward_folded(attn, ctx, fold=fold)
        return self.out.forward(attn, ctx, partials_ok=True)

    def forward(self, x, ctx, unit, writes, fold=None, state=None):
        if isinstance(x, Folded):
            folded, x = x, x.x
        else:
            folded = None
        kpages, vpages, block_table = ctx.unit_kv(unit)
        if self.prepared or self.gate_name is not None or not self.plain_softmax:
            return self._forward_prepared(x, ctx, writes, state, kpages, vpages, block_table, fold)
        fast_decode = ctx.is_decode and x.dtype == torch.bfloat16 and self.head_dim in DecodeKernels.HEAD_DIMS
        rotation = self.position.rotation() if self.position is not None else None
        tc = ctx.kernels.tensor_core if x.dtype == torch.bfloat16 else None
        # a rotation can ride in the decode attention kernel, or in the q|k|v product of a long prompt step
        fast_decode = fast_decode and not self.other_widths
        fusion = rotation if (fast_decode and rotation is not None and not self.own_store
                              and DecodeKernels.rotation_fusable(*rotation[1:])) else None
        fused_product = None
        if (tc is not None and writes and not fast_decode and not self.own_store and rotation is not None and x.shape[0] > tc.SKINNY_MAX_M
                and tc.rotation_fusable(self.head_dim, *rotation[1:]) and self.qkv.weight.dtype == torch.bfloat16
                and tc.takes(x, self.qkv.weight)):
            fused_product = rotation
        if fused_product is not None:
            # a long prompt step: the q|k|v product rotates and fills the cache in its own epilogue
            qkv = torch.empty((x.shape[0], self.n_heads * self.head_dim), dtype=x.dtype, device=x.device)
            tc.gemm_qkv_rope(x, self.qkv.weight, qkv, ctx.err_flag, ctx.tok_pos, ctx.tok_seq, block_table, fused_product[0],
                             kpages, vpages, self.n_heads, self.n_kv_heads, self.head_dim, fused_product[1], fused_product[2],
                             owed=(folded.sumsq, folded.width, folded.eps) if folded is not None else None)
        else:
            proj = self.qkv if writes else self.q_only
            qkv = proj.forward_folded(folded, ctx) if folded is not None else proj.forward(x, ctx)
            if fusion is None:
                self._store(qkv, ctx, rotation, self.n_kv_heads if writes else 0, kpages if writes else None,
                            vpages if writes else None, block_table)
        attn = self._attend(qkv, x, ctx, kpages, vpages, block_table, fast_decode, fusion, writes)
        if fold is not None:
            return self.out.forward_folded(attn, ctx, fold=fold)
        return self.out.forward(attn, ctx, partials_ok=True)


MIXERS.register("attention", Attention)

"""A short causal convolution over time, one filter per channel, with its last inputs as state.

y_t[c] = act(sum_j w[c, j] * in_{t - taps + 1 + j}[c] + bias[c]) with in = x (+ an input bias), the
column taps - 1 of w multiplies the row itself and rows in front of the sequence count as zero. A step sees only its
own rows, so the taps - 1 inputs before them are per-sequence state (float32), read by the step's
first rows and replaced at its end; a new sequence starts from zeros, which is the zero padding.
With `residual` the input is added to the result (y = in + conv(in)). Not a part of its own: mixers
and arrangements own one as they own a `Linear`, and publish its state under a name of theirs.
"""
from __future__ import annotations

import torch

from ..cache.needs import StateNeed
from ..weights.spec import TensorSpec


class CausalConv:
    graph_safe = True

    def prepare(self, max_positions: int, device) -> None:
        pass

    def elements_read_per_step(self) -> int:
        return self.width * self.taps + (self.width if self.bias_name is not None else 0)

    def __init__(self, names: list[str], channels: list[int], taps: int, bias_name: str | None = None,
                 residual: bool = False, act: str | None = None):
        if taps < 1:
            raise ValueError(f"a convolution needs at least one tap, got {taps}")
        if act not in (None, "silu"):
            raise ValueError(f"convolution activation {act!r}; known: silu")
        self.names, self.channels, self.taps = list(names), list(channels), int(taps)
        self.bias_name, self.residual, self.act = bias_name, residual, act
        self.width = sum(channels)
        self.weight = self.bias = None

    def tensor_specs(self):
        specs = [TensorSpec(n, (c, self.taps), init="conv_filter") for n, c in zip(self.names, self.channels)]
        if self.bias_name is not None:
            specs.append(TensorSpec(self.bias_name, (self.width,), init="bias"))
        return specs

    def bind(self, tensors, dtype, device):
        parts = [tensors[n] for n in self.names]
        self.weight = parts[0] if len(parts) == 1 else torch.cat(parts, dim=0).contiguous()
        self.bias = tensors[self.bias_name] if self.bias_name is not None else None

    @property
    def plain(self) -> bool:
        """Taps and nothing else: no bias, no added input, no activation (what a fused consumer takes over)."""
        return self.bias_name is None and not self.residual and self.act is None and self.taps > 1

    def state_need(self) -> StateNeed | None:
        return StateNeed((self.taps - 1, self.width), torch.float32) if self.taps > 1 else None

    def forward(self, x, state, ctx, out_dtype, in_bias=None, also=None):
        """x [T, width] (a view with unit column stride, float32 or the engine's dtype) -> [T, width] in
        `out_dtype`; `state`: the unit's tensor for this convolution (None with one tap); `also`: a
        second output of the engine's dtype to fill with the same values."""
        y = torch.empty((x.shape[0], self.width), dtype=out_dtype, device=x.device)
        ctx.kernels.seq.causal_conv(x, self.weight, state, ctx, y, self.taps, in_bias=in_bias, out_bias=self.bias,
                                    add_input=self.residual, act=self.act, y2=also)
        return y

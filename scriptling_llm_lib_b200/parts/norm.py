"""RMSNorm fused with the residual sum that precedes it.

y = (v / sqrt(mean(v^2) + eps)) * w with v = residual + delta; weight used as is, no bias, no mean
subtraction (float32_ops.go:159-172). The sum of squares, the division and the residual sum are
float32 whatever the engine's dtype.
"""
from __future__ import annotations

import torch

from dataclasses import dataclass
from typing import Any

from ..weights.spec import TensorSpec
from .base import NORMS, Folded, Norm


class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, width: int, eps: float, weight_name: str):
        self.width, self.eps, self.weight_name = width, float(eps), weight_name
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.weight_name, (self.width,), init="norm_weight")]

    def bind(self, tensors, dtype, device):
        self.weight = tensors[self.weight_name]
        self.weight_f32 = self.weight if self.weight.dtype == torch.float32 else self.weight.float()
        self._fold_memo = {}

    def fold_terms(self):
        return self.weight_f32, self.eps

    def forward(self, residual, delta, ctx, rows=None):
        if isinstance(delta, Folded):          # the product before this norm has done its work already
            return delta
        n = residual.shape[0] if rows is None else rows.shape[0]
        y = torch.empty((n, self.width), dtype=ctx.dtype, device=residual.device)
        if isinstance(delta, RmsNormedAddend):  # the addend's own norm, the sum and this norm in one pass
            ctx.kernels.gate.add_rms_normed(residual, delta.y, delta.weight, delta.eps, norm=(self.weight, self.eps, y), rows=rows)
            return y
        ctx.kernels.add_rmsnorm(residual, delta, rows, self.weight, y, self.eps)
        return y


@dataclass
class RmsNormedAddend:
    """An addend that joins the residual stream divided by its own root mean square: x += y / sqrt(mean(y^2) + eps) * weight.
    `y` is [T, width] (float32 or the engine's dtype) or float32 [P, T, width] partial sums, `weight` float32. The RMS norm
    that reads the stream next does both in one pass; `apply` does the sum by itself for a reader that is none."""
    y: Any
    weight: Any
    eps: float

    def apply(self, residual, ctx) -> None:
        ctx.kernels.gate.add_rms_normed(residual, self.y, self.weight, self.eps)


class WeightedNorm(Norm):
    """A norm with a weight and no bias in front of which the residual stream takes several
    addends, each with a coefficient: v = residual + sum c_i * a_i, then, with `center`,
    y = (v - mean(v)) / sqrt(mean((v - mean(v))^2) + eps) * w (layer norm), else
    y = v / sqrt(mean(v^2) + eps) * w. Sum, mean, variance and division are float32 whatever the
    engine's dtype. `delta`: None, one tensor [T, width] (coefficient 1), or a list of
    (tensor, coefficient); the tensors are float32 or of the engine's dtype. `out_dtype="float32"`
    keeps the normed rows in float32 for a reader that works on them before rounding (a short
    convolution in front of the mixer)."""
    graph_safe = True

    def __init__(self, width: int, eps: float, weight_name: str, center: bool = True, out_dtype: str | None = None):
        self.width, self.eps, self.weight_name, self.center = width, float(eps), weight_name, bool(center)
        self.out_dtype = {None: None, "float32": torch.float32}[out_dtype]
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.weight_name, (self.width,), init="norm_weight")]

    def bind(self, tensors, dtype, device):
        self.weight = tensors[self.weight_name]

    def forward(self, residual, delta, ctx, rows=None):
        addends = []
        for t, c in ([] if delta is None else [(delta, 1.0)] if isinstance(delta, torch.Tensor) else delta):
            if t.dim() == 3:                # partial sums of a product whose K range was split: each is an addend
                addends += [(t[i], c) for i in range(t.shape[0])]
            else:
                addends.append((t, c))
        n = residual.shape[0] if rows is None else rows.shape[0]
        y = torch.empty((n, self.width), dtype=self.out_dtype or ctx.dtype, device=residual.device)
        ctx.kernels.seq.add_norm(residual, addends, rows, self.weight, y, self.eps, self.center)
        return y


@dataclass
class WithRowVector:
    """A pending addend (`inner`: None or any form a norm takes) together with a vector float32 [width] that every row of
    the stream still has to take: x += inner; x += vector. The next reader of the stream adds both in its own pass."""
    inner: Any
    vector: Any


def take_into_stream(residual, delta, ctx, xb=None) -> None:
    """Adds a pending addend of any form into the stream by itself (no norm follows): None, a tensor in either form, a
    list of such tensors, an `RmsNormedAddend`, and any of them inside a `WithRowVector`. `xb` (the engine's dtype,
    [T, width]) receives the rounded stream."""
    vec = None
    if isinstance(delta, WithRowVector):
        delta, vec = delta.inner, delta.vector
    if isinstance(delta, RmsNormedAddend):
        ctx.kernels.gate.add_rms_normed(residual, delta.y, delta.weight, delta.eps, vec=vec)
        delta, vec = None, None
    if isinstance(delta, NormedAddend):
        raise ValueError("an addend that still has to pass a norm of its own is taken in by the norm that reads the stream next")
    addends = [] if delta is None else list(delta) if isinstance(delta, (list, tuple)) else [delta]
    if addends or vec is not None or xb is not None:
        ctx.kernels.gate.add_list_cast(residual, addends, xb, vec)


@dataclass
class NormedAddend:
    """A sublayer's output that passes a norm of its own before it joins the residual stream:
    x += norm(y). `y` is [T, width] (the engine's dtype or float32) or float32 [P, T, width] partial
    sums; `norm` is the part that owns weight, bias and slope. The norm that reads the stream next
    applies it while it forms the sum, so the addend is read once and never stored normed."""
    y: Any
    norm: "DynamicTanh"


class DynamicTanh(Norm):
    """A norm that takes no statistics of the row: y = tanh(alpha * v) * w + b, alpha one number,
    w and b vectors, every element on its own in float32. In front of a sublayer it reads
    v = residual + pending addend (the sum is kept); behind a sublayer it is only named in a
    `NormedAddend`, and the next reader of the stream does the work of both in one pass."""
    graph_safe = True

    def __init__(self, width: int, weight_name: str, bias_name: str, alpha_name: str):
        self.width, self.weight_name, self.bias_name, self.alpha_name = width, weight_name, bias_name, alpha_name
        self.weight = self.bias = None
        self.alpha = 1.0

    def tensor_specs(self):
        return [TensorSpec(self.weight_name, (self.width,), init="norm_weight"), TensorSpec(self.bias_name, (self.width,), init="bias"),
                TensorSpec(self.alpha_name, (), init="slope")]

    def elements_read_per_step(self) -> int:
        return 2 * self.width

    def bind(self, tensors, dtype, device):
        self.weight = tensors[self.weight_name].float().contiguous()
        self.bias = tensors[self.bias_name].float().contiguous()
        self.alpha = float(tensors[self.alpha_name].float().cpu())

    def terms(self):
        return self.weight, self.bias, self.alpha

    def forward(self, residual, delta, ctx, rows=None):
        """Besides a tensor and a `NormedAddend`, the pending addend may be an `RmsNormedAddend` (one kernel divides it by its
        root mean square, adds it and norms the row), a list of tensors, and any of these inside a `WithRowVector`."""
        vec = None
        if isinstance(delta, WithRowVector):
            delta, vec = delta.inner, delta.vector
        n = residual.shape[0] if rows is None else rows.shape[0]
        if isinstance(delta, RmsNormedAddend):
            y = torch.empty((n, self.width), dtype=ctx.dtype, device=residual.device)
            ctx.kernels.gate.add_rms_normed(residual, delta.y, delta.weight, delta.eps, rows=rows, vec=vec,
                                            dyt=(self.weight, self.bias, self.alpha, y))
            return y
        if isinstance(delta, (list, tuple)) or vec is not None:
            if isinstance(delta, NormedAddend):
                raise ValueError("a row vector does not travel with an addend that has a norm of its own")
            take_into_stream(residual, WithRowVector(delta, vec) if vec is not None else delta, ctx)
            delta = None
        addend, post = delta, None
        if isinstance(delta, NormedAddend):
            addend, post = delta.y, delta.norm.terms()
        n = residual.shape[0] if rows is None else rows.shape[0]
        y = torch.empty((n, self.width), dtype=ctx.dtype, device=residual.device)
        ctx.kernels.mix.dyt_add_norm(residual, addend, post, rows, self.weight, self.bias, self.alpha, y)
        return y


NORMS.register("rmsnorm", RMSNorm)
NORMS.register("dynamic_tanh", DynamicTanh)
NORMS.register("weighted_norm", WeightedNorm)

"""Dense SiLU-gated feed-forward: y = (silu(x Wg^T) * (x Wu^T)) Wd^T, no biases
(model_f32.go:476-493). Gate and up rows are stacked so one product serves both; when the
intermediate width is a multiple of 8 the stacked rows are kept in tiles of 16 (8 gate rows, the 8
matching up rows), so that one tensor-core tile holds both halves of a pair and the gate can be
applied before anything is written."""
from __future__ import annotations

import torch

from .base import FEED_FORWARDS, FeedForward, Folded
from .linear import Linear


class SwiGLU(FeedForward):
    graph_safe = True

    def __init__(self, hidden: int, intermediate: int, gate_name: str, up_name: str, down_name: str):
        self.hidden, self.intermediate = hidden, intermediate
        self.gate_up = Linear([gate_name, up_name], [intermediate, intermediate], hidden)
        self.down = Linear([down_name], [hidden], intermediate)

    def tensor_specs(self):
        return self.gate_up.tensor_specs() + self.down.tensor_specs()

    def bind(self, tensors, dtype, device):
        self.gate_up.bind(tensors, dtype, device)
        self.down.bind(tensors, dtype, device)
        F = self.intermediate
        self.tiled = F % 8 == 0
        if self.tiled:
            w = self.gate_up.weight
            self.gate_up.weight = w.view(2, F // 8, 8, self.hidden).permute(1, 0, 2, 3).reshape(2 * F, self.hidden).contiguous()

    def takes_folded(self, ctx, rows: int) -> bool:
        return self.tiled and self.gate_up.fold_path(ctx, rows, ctx.dtype) is not None

    def can_fold(self, ctx, rows: int) -> bool:
        return self.down.fold_path(ctx, rows, ctx.dtype, finishing=True) is not None

    def forward(self, x, ctx, fold=None):
        if isinstance(x, Folded) or fold is not None:
            plain = x.x if isinstance(x, Folded) else x
            rows = plain.shape[0]
            h = torch.empty((rows, self.intermediate), dtype=torch.bfloat16, device=plain.device)
            if isinstance(x, Folded) or (self.tiled and self.gate_up.fold_path(ctx, rows, ctx.dtype) is not None):
                self.gate_up.forward_folded(x, ctx, swiglu_out=h)
            else:
                h = self._hidden(x, ctx)
            return self.down.forward_folded(h, ctx, fold=fold) if fold is not None else self.down.forward(h, ctx, partials_ok=True)
        return self.down.forward(self._hidden(x, ctx), ctx, partials_ok=True)

    def _hidden(self, x, ctx):
        h = torch.empty((x.shape[0], self.intermediate), dtype=x.dtype, device=x.device)
        w = self.gate_up.weight
        fast = self.tiled and x.dtype == torch.bfloat16 and w.dtype == x.dtype
        if fast and ctx.kernels.tensor_core.prefers_skinny(x, w, "swiglu", ctx.engine.sm_count):
            ctx.kernels.tensor_core.gemm_skinny(x, w, h, ctx.err_flag, swiglu=True)
        elif fast and ctx.kernels.decode.prefers(x, w, ctx.engine.sm_count):
            ctx.kernels.decode.gemm_small_m(x, w, h, swiglu=True)
        elif fast and ctx.kernels.tensor_core.takes(x, w):
            ctx.kernels.tensor_core.gemm(x, w, h, ctx.err_flag, swiglu=True)
        else:
            gu = self.gate_up.forward(x, ctx)
            ctx.kernels.swiglu(gu, h, tiled=self.tiled)
        return h


class ClampedGLU(FeedForward):
    """Dense feed-forward with the clamped gate (absent in the reference): g = min(Wg x, limit), u = clamp(Wu x, -limit, limit),
    y = Wd (g * sigmoid(alpha g) * (u + 1)). Gate and up rows are stacked into one product; in bfloat16 with widths in
    multiples of 8 they are kept in tiles of 16 (8 gate rows, their 8 up rows), and a long step runs the grouped tensor-core
    product with one group, whose epilogue applies the gate on the float sums and writes the inner vector only. Otherwise
    the product's sums pass the gate in a kernel of its own."""
    graph_safe = True

    def __init__(self, hidden: int, intermediate: int, gate_name: str, up_name: str, down_name: str, limit: float,
                 alpha: float = 1.702):
        if not float(limit) > 0:
            raise ValueError(f"the clamped gate needs a positive limit, got {limit}")
        self.hidden, self.intermediate, self.glu = hidden, intermediate, (float(limit), float(alpha))
        self.gate_up = Linear([gate_name, up_name], [intermediate, intermediate], hidden)
        self.down = Linear([down_name], [hidden], intermediate)

    def tensor_specs(self):
        return self.gate_up.tensor_specs() + self.down.tensor_specs()

    def bind(self, tensors, dtype, device):
        self.gate_up.bind(tensors, dtype, device)
        self.down.bind(tensors, dtype, device)
        F = self.intermediate
        self.tiled = dtype == torch.bfloat16 and F % 8 == 0 and self.hidden % 8 == 0
        if self.tiled:
            w = self.gate_up.weight
            self.gate_up.weight = w.view(2, F // 8, 8, self.hidden).permute(1, 0, 2, 3).reshape(2 * F, self.hidden).contiguous()
        self.one_group = torch.zeros((128,), dtype=torch.int32, device=device)      # the one group every row tile belongs to

    def forward(self, x, ctx):
        T, F = x.shape[0], self.intermediate
        h = torch.empty((T, F), dtype=x.dtype, device=x.device)
        tc = ctx.kernels.tensor_core if x.dtype == torch.bfloat16 else None
        if self.tiled and tc is not None and T > tc.SKINNY_MAX_M and x.data_ptr() % 16 == 0 and x.is_contiguous():
            tiles = -(-T // 128)
            if self.one_group.shape[0] < tiles:
                self.one_group = torch.zeros((tiles,), dtype=torch.int32, device=x.device)
            tc.gemm_grouped(x, self.gate_up.weight.unsqueeze(0), h, self.one_group[:tiles], ctx.err_flag, glu=self.glu)
        else:
            gu = self.gate_up.forward(x, ctx)
            ctx.kernels.mix.glu_clamp(gu, h, self.glu[0], self.glu[1], tiled=self.tiled)
        return self.down.forward(h, ctx, partials_ok=True)


FEED_FORWARDS.register("swiglu", SwiGLU)
FEED_FORWARDS.register("clamped_glu", ClampedGLU)

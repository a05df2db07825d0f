"""A per-layer input from the token itself, gated by the residual stream.

Every token has a second, narrow embedding e (a row of a table shared by all layers, of which layer i reads
the columns [i * dim, (i + 1) * dim)). With x the residual stream as it stands behind the layer's sublayers:

    g = gelu_tanh(Wgate x) * e        [dim]
    y = Wproj g                       [width]
    x += y / sqrt(mean(y^2) + eps) * w

The last line is left pending (`RmsNormedAddend`): the norm that reads the stream next does it in its own pass.
The stream's sum and the norm are float32; the two products are the library's (in the engine's dtype on the
stream rounded once, with float32 sums), the second one leaving float32. The table is one tensor for the
model: the first layer that asks for it owns it in the weight list, the others name it as theirs (`owns_table`).
Not in the reference.
"""
from __future__ import annotations

import torch

from ..weights.spec import TensorSpec
from .base import STREAM_INPUTS, StreamInput
from .linear import Linear
from .norm import RmsNormedAddend, take_into_stream


class TokenSideInput(StreamInput):
    graph_safe = True

    def __init__(self, width: int, dim: int, vocab: int, table_name: str, table_width: int, column: int, gate_name: str,
                 proj_name: str, norm_name: str, eps: float, owns_table: bool = True):
        if dim < 1 or column < 0 or column + dim > table_width:
            raise ValueError(f"columns {column}..{column + dim} are outside a table of width {table_width}")
        self.width, self.dim, self.vocab, self.eps = width, dim, vocab, float(eps)
        self.table_name, self.table_width, self.column, self.owns_table = table_name, table_width, column, owns_table
        self.norm_name = norm_name
        self.gate = Linear([gate_name], [dim], width)
        self.proj = Linear([proj_name], [width], dim)
        self.table = self.weight = None

    def tensor_specs(self):
        specs = [TensorSpec(self.table_name, (self.vocab, self.table_width))] if self.owns_table else []
        return specs + self.gate.tensor_specs() + self.proj.tensor_specs() + [TensorSpec(self.norm_name, (self.width,), init="norm_weight")]

    def elements_read_per_step(self) -> int:
        return 2 * self.dim * self.width + self.width      # a step reads a table row per token, not the table

    def bind(self, tensors, dtype, device):
        self.gate.bind(tensors, dtype, device)
        self.proj.bind(tensors, dtype, device)
        self.table = tensors[self.table_name]
        self.weight = tensors[self.norm_name].float().contiguous()
        if self.table.dtype != dtype:
            raise ValueError(f"the table {self.table_name} is {self.table.dtype}, the engine runs in {dtype}")

    def forward(self, residual, delta, ctx):
        k = ctx.kernels.gate
        T = residual.shape[0]
        xb = torch.empty((T, self.width), dtype=ctx.dtype, device=residual.device)
        if delta is None or isinstance(delta, torch.Tensor):
            k.add_cast(residual, delta, xb)                              # the stream takes the sublayer's output; xb = its rounding
        else:                                                            # several addends, or one of the composite forms
            take_into_stream(residual, delta, ctx, xb=xb)
        a = self.gate.forward(xb, ctx)
        g = torch.empty((T, self.dim), dtype=ctx.dtype, device=residual.device)
        k.gelu_mul_rows(a, ctx.token_ids, self.table, self.column, g)
        y = self.proj.forward(g, ctx, out_dtype=torch.float32, partials_ok=True)
        return RmsNormedAddend(y, self.weight, self.eps)      # the next reader's norm adds it while it norms


STREAM_INPUTS.register("token_side", TokenSideInput)

"""A vector that every row of the residual stream takes at a point between two layers.

A model that goes through a run of its layers several times with the same weights tells the passes apart by a stored
vector each: before pass t's first layer, x += V[t] on every row, V [passes, width]. The part owns the whole table (the
first to ask names it in the weight list, `owns_table`), and an instance stands for one row of it. Nothing is computed
here: the vector travels with whatever is still pending (`WithRowVector`) and the norm that reads the stream next adds
both in its own pass. The sum is float32. Not in the reference.
"""
from __future__ import annotations

from ..weights.spec import TensorSpec
from .base import STREAM_INPUTS, StreamInput
from .norm import WithRowVector


class PassVector(StreamInput):
    graph_safe = True

    def __init__(self, width: int, table_name: str, rows: int, row: int, owns_table: bool = True):
        if not 0 <= row < rows:
            raise ValueError(f"row {row} of a table of {rows} rows")
        self.width, self.table_name, self.rows, self.row, self.owns_table = width, table_name, rows, row, owns_table
        self.vector = None

    def tensor_specs(self):
        return [TensorSpec(self.table_name, (self.rows, self.width), init="bias")] if self.owns_table else []

    def elements_read_per_step(self) -> int:
        return self.width

    def bind(self, tensors, dtype, device):
        self.vector = tensors[self.table_name][self.row].float().contiguous()

    def forward(self, residual, delta, ctx):
        if isinstance(delta, WithRowVector):          # two vectors in a row: one sum
            return WithRowVector(delta.inner, delta.vector + self.vector)
        return WithRowVector(delta, self.vector)


STREAM_INPUTS.register("pass_vector", PassVector)

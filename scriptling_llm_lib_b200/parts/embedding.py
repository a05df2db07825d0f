"""Token embedding and output head.

x[i, :] = E[id_i, :], no scaling (model_f32.go:363-369); logits = n W^T with W the embedding when
the head is tied (model_f32.go:147-162, :519-524). The reference skips ids outside the table and
leaves stale data in the row; here such an id is an error before anything runs. Both are parts
like the others, named in a layout by kind ("token_embedding", "linear_head"): a model that scales
its embedding or caps its logits registers parts of its own.
"""
from __future__ import annotations

import torch

from ..weights.spec import TensorSpec
from .base import EMBEDDINGS, HEADS, Embedding, Head, PartSpec
from .linear import Linear


class TokenEmbedding(Embedding):
    def __init__(self, vocab: int, width: int, name: str):
        self.vocab, self.width, self.name = vocab, width, name
        self.table = None

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.vocab, self.width))]

    def elements_read_per_step(self) -> int:
        return 0                                    # a step reads one row per token, not the table

    def bind(self, tensors, dtype, device):
        self.table = tensors[self.name]

    def forward(self, ids, ctx):
        out = torch.empty((ids.shape[0], self.width), dtype=torch.float32, device=ids.device)
        if self.table.dtype == ctx.dtype:
            ctx.kernels.embed_rows(ids, self.table, out, ctx.err_flag)
        else:
            ctx.kernels_f32.embed_rows(ids, self.table, out, ctx.err_flag)
        return out


class PairHashEmbedding(Embedding):
    """x = E[token] + P[r]: a second table P [buckets + 1, width] is looked up by the pair (previous token, token),
    r = (previous * mul_prev + token * mul_cur) mod buckets, and by its last row, r = buckets, for a sequence's first token
    (absent in the reference). The previous token of a step's first row is per-sequence state: one int32 per slot
    (`state_need`), read and then set to the run's last token by the embedding kernel itself, so prompts in portions,
    decode steps and replayed steps all find it on the device."""

    def __init__(self, vocab: int, width: int, name: str, pair_name: str, buckets: int, mul_prev: int, mul_cur: int):
        if buckets < 1 or mul_prev < 0 or mul_cur < 0:
            raise ValueError(f"a pair table of {buckets} buckets with multipliers {mul_prev}, {mul_cur}")
        self.vocab, self.width, self.name, self.pair_name = vocab, width, name, pair_name
        self.buckets, self.mul_prev, self.mul_cur = int(buckets), int(mul_prev), int(mul_cur)
        self.table = self.pair_table = None

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.vocab, self.width)), TensorSpec(self.pair_name, (self.buckets + 1, self.width))]

    def elements_read_per_step(self) -> int:
        return 0                                    # two rows per token, not the tables

    def state_need(self):
        from ..cache.needs import StateNeed
        return StateNeed((), torch.int32)

    def bind(self, tensors, dtype, device):
        self.table, self.pair_table = tensors[self.name], tensors[self.pair_name]
        if self.table.dtype != self.pair_table.dtype:
            raise ValueError(f"{self.name} and {self.pair_name} are stored in different precisions")

    def forward(self, ids, ctx):
        out = torch.empty((ids.shape[0], self.width), dtype=torch.float32, device=ids.device)
        k = ctx.kernels if self.table.dtype == ctx.dtype else ctx.kernels_f32
        k.embed_pair_rows(ids, ctx, self.table, self.pair_table, self.buckets, self.mul_prev, self.mul_cur,
                          ctx.unit_state(EMBEDDING_STATE), out, ctx.err_flag)
        return out


EMBEDDING_STATE = "embedding"      # the key of the embedding's per-sequence state among the cache units' states


class OutputHead(Head):
    """Logits in float32 for the rows it is given. `tied`: the matrix is another part's tensor (the
    embedding's), named by `weight_name`, and is not asked of the weight file a second time. `softcap` (absent in the
    reference): the logits leave as cap * tanh(logits / cap). `scale` (absent in the reference): the logits are multiplied by
    it (before a cap)."""

    def __init__(self, vocab: int, width: int, weight_name: str, tied: bool = False, softcap: float | None = None,
                 scale: float | None = None):
        self.vocab, self.width, self.tied = vocab, width, tied
        self.scale = float(scale) if scale is not None else 1.0
        self.softcap = float(softcap) if softcap else None
        if self.softcap is not None and not self.softcap > 0:
            raise ValueError(f"a cap on the logits must be positive, got {softcap}")
        self.linear = Linear([weight_name], [vocab], width)

    def tensor_specs(self):
        return [] if self.tied else self.linear.tensor_specs()

    def elements_read_per_step(self) -> int:
        return self.vocab * self.width

    def bind(self, tensors, dtype, device):
        self.linear.bind(tensors, dtype, device)

    def forward(self, normed, ctx):
        logits = self.linear.forward(normed, ctx, out_dtype=torch.float32)
        if self.softcap is not None or self.scale != 1.0:
            ctx.kernels.gate.softcap(logits, self.softcap, self.scale)
        return logits


EMBEDDINGS.register("token_embedding", TokenEmbedding)
EMBEDDINGS.register("pair_hash_embedding", PairHashEmbedding)
HEADS.register("linear_head", OutputHead)


def token_embedding(vocab: int, width: int, name: str) -> PartSpec:
    return PartSpec("token_embedding", dict(vocab=vocab, width=width, name=name))


def linear_head(vocab: int, width: int, weight_name: str, tied: bool = False, softcap: float | None = None,
                scale: float | None = None) -> PartSpec:
    params = dict(vocab=vocab, width=width, weight_name=weight_name, tied=tied)
    if softcap:
        params["softcap"] = softcap
    if scale is not None and scale != 1.0:
        params["scale"] = scale
    return PartSpec("linear_head", params)

"""Causal softmax attention whose keys and values are made from a cached latent.

From the mixer's input h: q = Wq h, per head [dim unrotated | rot_dim rotated] dims. Wdkv h has
kv_rank + rot_dim rows: the first kv_rank, divided by their root mean square and multiplied by a
weight, are the latent c; the last rot_dim are a key part that all heads share. Head i's key is
[Wuk_i c | shared part], its value Wuv_i c; the score is (q . k) * scale, the mask causal, the
softmax ordinary, and Wo maps the heads' outputs back. A position encoding (a rotation by a table)
turns the rot_dim part of every query head and the shared key part; values are not turned.

The cache holds c and the rotated key part and nothing else: one vector of kv_rank + rot_dim per
position, whatever the number of heads (a cache unit with one key "head" of that width and no value storage). Keys
and values are never formed per position. Since q_i . (Wuk_i c) = (Wuk_i^T q_i) . c, a head asks
the cached vectors with [Wuk_i^T q_i | q_rot] directly, sums the latents with the softmax weights,
and applies Wuv_i once to that sum. All heads of a row read the same cached rows. That is the form
of decode steps and of portions that land on a cache. A prompt step whose sequences all start at
position 0 forms keys and values per head for its own rows instead (two products over the step's
latents) and runs the library's attention kernel for keys and values of one width on them: fewer
products per query and key than asking the latent, which is wider than a head.

A layer built with `shares_cache=True` has no Wdkv: it runs with `writes=False` on the unit another
latent-attention layer of the same widths and rotation wrote, with its own Wq, Wuk, Wuv and Wo.

Three options. `q_rank`: the queries go through a latent of their own, c_q = (Wdq h) / rms * w and q = Wuq c_q (the
down-projection leaves float32 sums, the norm is float32, and `q_name` is not used). `pairing="half"`: the rotated part
turns dim i with dim i + rot / 2 instead of neighbours. `gate_name`: a matrix [n_heads, hidden] on the mixer's input; head
i's output is multiplied by the sigmoid of its logit before Wo (the logits ride in the down-projection's product).
`prompt_kernel="tensor"`: in bfloat16 the per-head form of a prompt runs on the mma.sync attention kernel that takes keys and
values of different widths (rows padded with zeros to the widths it is built for) instead of the float32 tiled kernel; the
weights then enter the product with the values rounded to bfloat16.

The products run in the engine's dtype and the cache holds it; the latent's norm, the rotation,
the absorbed queries, scores, softmax and sums over the latent are float32.
"""
from __future__ import annotations

import torch

from ..cache.needs import PAGE, CacheNeed
from ..weights.spec import TensorSpec
from .base import MIXERS, POSITION_ENCODINGS, Mixer, PartSpec
from .linear import Linear


class LatentAttention(Mixer):
    graph_safe = True
    MAX_RANK = 1024          # the kernel keeps a lane's share of the latent sum in registers

    def __init__(self, hidden: int, n_heads: int, dim: int, rot_dim: int, v_dim: int, kv_rank: int, scale: float,
                 position: PartSpec | None, norm_eps: float, q_name: str | None, uk_name: str, uv_name: str, o_name: str,
                 dkv_name: str | None = None, dkv_norm_name: str | None = None, shares_cache: bool = False,
                 q_rank: int | None = None, dq_name: str | None = None, dq_norm_name: str | None = None, uq_name: str | None = None,
                 gate_name: str | None = None, prompt_kernel: str = "float32"):
        if kv_rank < 1 or kv_rank > self.MAX_RANK:
            raise ValueError(f"latent of width {kv_rank}: the attention kernel takes 1..{self.MAX_RANK}")
        if not shares_cache and (dkv_name is None or dkv_norm_name is None):
            raise ValueError("a latent-attention layer with a cache of its own needs the down-projection and its norm weight")
        self.hidden, self.H, self.D, self.P, self.V, self.R = hidden, n_heads, dim, rot_dim, v_dim, kv_rank
        self.scale, self.eps, self.shares_cache = float(scale), float(norm_eps), bool(shares_cache)
        self.position = POSITION_ENCODINGS.build(position) if position is not None else None
        qw = n_heads * (dim + rot_dim)
        self.q_width = qw
        self.q_rank = int(q_rank) if q_rank else None
        self.gate_name, self.dq_norm_name = gate_name, dq_norm_name
        if self.q_rank is not None:
            if dq_name is None or dq_norm_name is None or uq_name is None:
                raise ValueError("queries through a latent need its down-projection, norm weight and up-projection")
            self.q_down = Linear([dq_name], [self.q_rank], hidden)
            self.q_up = Linear([uq_name], [qw], self.q_rank)
            names, widths = [], []
        else:
            if q_name is None:
                raise ValueError("a latent-attention layer needs a query projection, direct or through a latent")
            self.q_down = self.q_up = None
            names, widths = [q_name], [qw]
        self.q_cols = widths[0] if widths else 0           # columns of the stacked product that are queries
        if not shares_cache:
            names, widths = names + [dkv_name], widths + [kv_rank + rot_dim]
        if gate_name is not None:
            names, widths = names + [gate_name], widths + [n_heads]
        self.proj = Linear(names, widths, hidden) if names else None
        self.out = Linear([o_name], [hidden], n_heads * v_dim)
        self.kv_up = Linear([uk_name, uv_name], [n_heads * dim, n_heads * v_dim], kv_rank)
        if prompt_kernel not in ("float32", "tensor"):
            raise ValueError(f"prompt kernel {prompt_kernel!r}; known: float32, tensor")
        self.prompt_kernel = prompt_kernel
        self.hd = (max(dim + rot_dim, v_dim) + 3) // 4 * 4      # one width for keys, values and queries of the per-head form
        self.mma = None                                         # (key width, value width) of the tensor-core prompt kernel, once bound
        self.uk_name, self.uv_name, self.dkv_norm_name = uk_name, uv_name, dkv_norm_name

    def tensor_specs(self):
        specs = (self.proj.tensor_specs() if self.proj is not None else []) + self.out.tensor_specs()
        if self.q_rank is not None:
            specs += self.q_down.tensor_specs() + self.q_up.tensor_specs() + [TensorSpec(self.dq_norm_name, (self.q_rank,), init="norm_weight")]
        specs += [
            TensorSpec(self.uk_name, (self.H * self.D, self.R)), TensorSpec(self.uv_name, (self.H * self.V, self.R))]
        if not self.shares_cache:
            specs.append(TensorSpec(self.dkv_norm_name, (self.R,), init="norm_weight"))
        return specs

    def bind(self, tensors, dtype, device):
        if self.proj is not None:
            self.proj.bind(tensors, dtype, device)
        if self.q_rank is not None:
            self.q_down.bind(tensors, dtype, device)
            self.q_up.bind(tensors, dtype, device)
            self.q_norm_w = tensors[self.dq_norm_name].float().contiguous()
        self.out.bind(tensors, dtype, device)
        self.wuk, self.wuv = tensors[self.uk_name], tensors[self.uv_name]
        self.kv_up.bind(tensors, dtype, device)
        if self.prompt_kernel == "tensor" and dtype == torch.bfloat16:
            from ..csrc.bindings import PrefillAttentionMMA
            self.mma = PrefillAttentionMMA.widths_for(self.D + self.P, self.V)
            if self.mma is not None:                            # rows padded with zeros up to the widths that kernel is built for
                self.hd = max(self.mma)
        # the output matrix with zero columns where the per-head form pads a head's values to `hd`
        if self.hd != self.V:
            w = self.out.weight
            wide = torch.zeros((w.shape[0], self.H, self.hd), dtype=w.dtype, device=w.device)
            wide[:, :, :self.V] = w.view(w.shape[0], self.H, self.V)
            self.out_wide = self.out.rows(0, w.shape[0])
            self.out_wide.in_features = self.H * self.hd
            self.out_wide.weight = wide.view(w.shape[0], self.H * self.hd)
        else:
            self.out_wide = self.out
        self.norm_w = None if self.shares_cache else tensors[self.dkv_norm_name].float().contiguous()

    def prepare(self, max_positions, device):
        if self.position is not None:
            self.position.prepare(max_positions, device)

    def cache_need(self):
        return CacheNeed("full", 1, self.R + self.P, None, v_dim=0)

    def splits(self, ctx) -> int:
        """Over how many blocks a row's keys are split: one in a prompt step (its rows fill the GPU), in a
        decode step enough for about two blocks per SM, at most one per 32 keys of the longest sequence."""
        if not ctx.is_decode:
            return 1
        blocks = ctx.n_seqs * -(-self.H // 8)
        return max(1, min(-(-2 * ctx.engine.sm_count // blocks), ctx.max_pages * PAGE // 32, 64))

    PER_HEAD_MIN_ROWS = 32       # prompts from position 0 with at least this many rows form keys and values per head

    def _tables(self, ctx):
        """Pages of their own for the per-head keys and values of a prompt step: every sequence's positions from a
        page border on; one table for all layers of the step."""
        made = ctx.scratch.get("latent_heads_table")
        if made is None:
            import numpy as np
            per = [-(-n // PAGE) for n in ctx.seq_lens_host]
            table = np.zeros((len(per), max(per)), dtype=np.int32)
            at = 0
            for b, n in enumerate(per):
                table[b, :n] = np.arange(at, at + n)
                at += n
            made = (torch.from_numpy(table).pin_memory().to(ctx.slots.device, non_blocking=True), at)
            ctx.scratch["latent_heads_table"] = made
        return made

    def _finish(self, attn, gate, width, out, ctx):
        """The gate per head (where the layer has one) and the output product."""
        if gate is not None:
            ctx.kernels.gate.head_gate(attn, gate, self.H, width)
        return out.forward(attn, ctx, partials_ok=True)

    def _per_head(self, q, ctx, pages, block_table, gate=None):
        """The prompt from position 0: keys [Wuk c | rotated part] and values Wuv c per head for the step's rows, then
        the library's attention kernel for keys and values of one width over pages of their own. Costs
        (dim + rot_dim + v_dim) products per query, key and head instead of (2 kv_rank + rot_dim)."""
        k = ctx.kernels.mix
        T, dev = q.shape[0], q.device
        dense = torch.empty((T, self.R + self.P), dtype=q.dtype, device=dev)
        k.latent_gather(pages, ctx, block_table, dense)
        kv = self.kv_up.forward(dense[:, :self.R], ctx)                       # [T, H dim | H v_dim]
        table, n_pages = self._tables(ctx)
        kt = torch.empty((n_pages, self.H, PAGE, self.hd), dtype=q.dtype, device=dev)
        vt = torch.empty((n_pages, self.H, PAGE, self.hd), dtype=q.dtype, device=dev)
        qt = torch.empty((T, self.H * self.hd), dtype=q.dtype, device=dev)
        k.latent_heads(q, kv, dense, self.R, ctx, table, kt, vt, qt, self.H, self.D, self.P, self.V, self.hd)
        attn = torch.empty((T, self.H * self.hd), dtype=q.dtype, device=dev)
        if self.mma is not None:
            ctx.kernels.prefill_attention_mma.attn(qt, self.hd, attn, self.hd, ctx.seq_start, ctx.seq_pos0, table, kt, vt, ctx.n_seqs,
                                                   ctx.max_new, self.H, self.H, self.mma[0], self.mma[1], None, self.scale)
        else:
            ctx.kernels.attn_paged(qt, attn, ctx.seq_start, ctx.seq_pos0, table, kt, vt, ctx.n_seqs, ctx.max_new, self.H, self.H,
                                   self.hd, None, self.scale)
        return self._finish(attn, gate, self.hd, self.out_wide, ctx)

    def forward(self, x, ctx, unit, writes):
        if writes == self.shares_cache:
            raise ValueError("a latent-attention layer writes the cache unit exactly when it has a down-projection of its own")
        k = ctx.kernels.mix
        pages, _, block_table = ctx.unit_kv(unit)
        T = x.shape[0]
        proj = self.proj.forward(x, ctx) if self.proj is not None else None     # [T, (q |) (latent and key part, raw |) (gate logits)]
        if self.q_rank is not None:                                              # queries through their own normed latent
            cq = self.q_down.forward(x, ctx, out_dtype=torch.float32)
            cqn = torch.empty((T, self.q_rank), dtype=x.dtype, device=x.device)
            ctx.kernels.add_rmsnorm(cq, None, None, self.q_norm_w, cqn, self.eps)
            q = self.q_up.forward(cqn, ctx)
        else:
            q = proj[:, :self.q_width]
        at = self.q_cols
        dkv = None
        if writes:
            dkv = proj[:, at:at + self.R + self.P]
            at += self.R + self.P
        gate = proj[:, at:at + self.H] if self.gate_name is not None else None
        table, rot, half = None, 0, False
        if self.position is not None:
            table, rot, interleaved = self.position.rotation()
            half = not interleaved
        k.latent_store(q, self.H, self.D, dkv, self.norm_w, self.eps, table, rot, ctx,
                       block_table, pages if writes else None, self.R, self.P, half=half)
        if ctx.from_start and not ctx.is_decode and ctx.max_new >= self.PER_HEAD_MIN_ROWS:
            return self._per_head(q, ctx, pages, block_table, gate)
        qa = torch.empty((T, self.H, self.R + self.P), dtype=torch.float32, device=x.device)
        k.latent_absorb(q, self.wuk, qa, self.H, self.D, self.P, self.R, self.scale)
        n_split = self.splits(ctx)
        part = torch.empty((T, self.H, n_split, self.R + 2), dtype=torch.float32, device=x.device)
        k.latent_attn(qa, pages, ctx, block_table, part, self.H, self.R, self.P, n_split)
        attn = torch.empty((T, self.H * self.V), dtype=x.dtype, device=x.device)
        olat = torch.empty((T, self.H, self.R), dtype=torch.float32, device=x.device)
        k.latent_expand(part, olat, self.wuv, attn, self.H, self.V, self.R, n_split)
        return self._finish(attn, gate, self.V, self.out, ctx)


MIXERS.register("latent_attention", LatentAttention)

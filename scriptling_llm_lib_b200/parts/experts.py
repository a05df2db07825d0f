"""Feed-forwards with one activation, dense or routed to a few of many small experts.

`act_feed_forward`: y = Wdown act(Wup x), no gate, no biases; act is the tanh form of gelu, the
square of relu, or silu.

`routed_experts`: `experts` such feed-forwards (act = relu^2 by default); a token runs `top` of
them. Router: z = Wr x with float32 sums (one of the library's products writing float32) and
s = sigmoid(z). Two scores per expert follow: c = s + correction (a stored vector) decides who is
picked, s alone decides how much a picked expert counts. The experts are cut into `n_groups` runs
of equal length; a run is rated by its best two c added up, the `keep_groups` best-rated runs stay
open, and every expert outside them is out of the race (its c is taken as -inf, so that a negative
c inside an open run still beats it). Among the open experts the `top` with the highest c are picked,
and expert e counts with s_e / (sum of the picked s + 1e-20) * scale. The output is the sum of the
picked experts' outputs with those factors.

Two more choices. `router="top_softmax"`: z = Wr x + bias (the stored vector is a bias on the logits here), the
`top` experts with the largest z are picked, and they count with the softmax over the picked logits alone (no
runs, no scale). `act="clamped_glu"`: an expert has a gate and an up matrix; with g = min(Wg x, limit) and
u = clamp(Wu x, -limit, limit) its inner vector is g * sigmoid(alpha g) * (u + 1), alpha = 1.702 unless
given. Gate and up rows are stacked per expert ([experts, 2 ff, hidden]) and multiplied in one pass; in bfloat16
with widths the tensor cores take they are stacked in tiles of 16 (8 gate rows, their 8 up rows), so that a long
step's grouped product applies the gate in its epilogue and writes the inner vector only.

Three more. `router="grouped_softmax"`: the scores are the softmax of z over ALL experts; a run of experts is rated by its
best score alone, the `keep_groups` best runs stay open, the `top` open experts with the highest scores are picked, and
they count with their scores as they are, not renormalised (times `scale`); no stored correction. `act="silu_glu"`: an
expert's inner vector is silu(Wg x) * (Wu x), the gate without a clamp (stacked and tiled like the clamped one).
`shared`: a feed-forward (a `PartSpec` of the FEED_FORWARDS registry) that every token runs beside its chosen experts; the
part then answers with a list of two addends, the routed sum and the shared expert's output.

The experts' matrices are stacked [experts, ff, hidden] and [experts, hidden, ff]. A step of few
rows runs every (token, chosen expert) pair by itself (each streams its expert's matrices once); a
longer step groups the pairs by expert on the device and runs tiles of rows per expert: in bfloat16
on the tensor cores (every expert's rows start at a multiple of 128, the product kernel looks up
each tile's expert, the weighted sum over a token's choices is a pass of its own), else on the FMA
units. All launch the same work whatever the router chose, so a decode step can be captured. The
weighted outputs leave as float32: partial sums [top, T, hidden], one per choice, which the next
reader of the residual stream adds in a fixed order, or the sum itself.
"""
from __future__ import annotations

import torch

from ..weights.spec import TensorSpec
from .base import FEED_FORWARDS, FeedForward
from .linear import Linear

ACTS = ("gelu_tanh", "relu_squared", "silu")
ROUTERS = ("grouped_sigmoid", "top_softmax", "grouped_softmax")


class ActFeedForward(FeedForward):
    graph_safe = True

    def __init__(self, hidden: int, intermediate: int, up_name: str, down_name: str, act: str = "gelu_tanh"):
        if act not in ACTS:
            raise ValueError(f"activation {act!r}; known: {', '.join(ACTS)}")
        self.hidden, self.intermediate, self.act = hidden, intermediate, act
        self.up = Linear([up_name], [intermediate], hidden)
        self.down = Linear([down_name], [hidden], intermediate)

    def tensor_specs(self):
        return self.up.tensor_specs() + self.down.tensor_specs()

    def bind(self, tensors, dtype, device):
        self.up.bind(tensors, dtype, device)
        self.down.bind(tensors, dtype, device)

    def forward(self, x, ctx):
        w = self.up.weight
        if x.dtype == torch.bfloat16 and w.dtype == x.dtype:
            tc = ctx.kernels.tensor_core
            if x.shape[0] > tc.SKINNY_MAX_M and tc.takes(x, w) and not ctx.kernels.decode.prefers(x, w, ctx.engine.sm_count):
                # a long step: the activation rides in the tensor-core product's epilogue, on the float sums
                h = torch.empty((x.shape[0], self.intermediate), dtype=x.dtype, device=x.device)
                tc.gemm_act(x, w, h, ctx.err_flag, self.act)
                return self.down.forward(h, ctx, partials_ok=True)
        h = self.up.forward(x, ctx)
        ctx.kernels.mix.act_inplace(h, self.act)
        return self.down.forward(h, ctx, partials_ok=True)


class RoutedExperts(FeedForward):
    graph_safe = True
    PAIRS_ONE_BY_ONE = 64        # up to this many (token, expert) pairs in a step each pair runs by itself

    def __init__(self, hidden: int, intermediate: int, experts: int, top: int, n_groups: int, keep_groups: int, scale: float,
                 router_name: str, correction_name: str | None, up_names: list, down_names: list, act: str = "relu_squared",
                 router: str = "grouped_sigmoid", gate_names: list | None = None, limit: float | None = None,
                 alpha: float = 1.702, shared=None):
        if act not in ("relu_squared", "clamped_glu", "silu_glu"):
            raise ValueError("the experts' kernels apply the square of relu, the clamped gate (clamped_glu) or the plain gate (silu_glu)")
        if router not in ROUTERS:
            raise ValueError(f"router {router!r}; known: {', '.join(ROUTERS)}")
        if len(up_names) != experts or len(down_names) != experts:
            raise ValueError(f"{experts} experts need as many up and down matrices")
        self.glu = None
        if act == "clamped_glu":
            if gate_names is None or len(gate_names) != experts or limit is None or not float(limit) > 0:
                raise ValueError("gated experts need a gate matrix each and a positive limit")
            self.glu = (float(limit), float(alpha))
        elif act == "silu_glu":
            if gate_names is None or len(gate_names) != experts:
                raise ValueError("gated experts need a gate matrix each")
            self.glu = (0.0, 1.0)           # a limit of 0: the kernels' word for the gate without a clamp
        self.gate_names = list(gate_names) if self.glu is not None else None
        self.router_kind = router
        self.top_softmax = router == "top_softmax"
        if self.top_softmax and n_groups != 1:
            raise ValueError("the top_softmax router knows no runs of experts")
        if router == "grouped_sigmoid" and correction_name is None:
            raise ValueError("the grouped_sigmoid router needs its correction")
        self.shared = FEED_FORWARDS.build(shared) if shared is not None else None
        if n_groups < 1 or experts % n_groups or not 1 <= keep_groups <= n_groups:
            raise ValueError(f"{experts} experts cannot form {n_groups} equal groups of which {keep_groups} are kept")
        if not 1 <= top <= keep_groups * (experts // n_groups):
            raise ValueError(f"{top} experts a token cannot come out of {keep_groups} groups of {experts // n_groups}")
        self.hidden, self.F, self.E, self.top = hidden, intermediate, experts, top
        self.n_groups, self.keep, self.scale = n_groups, keep_groups, float(scale)
        self.router_name, self.correction_name = router_name, correction_name
        self.router = Linear([router_name], [experts], hidden)
        self.up_names, self.down_names = list(up_names), list(down_names)

    def tensor_specs(self):
        specs = self.router.tensor_specs()
        if self.correction_name is not None:
            specs.append(TensorSpec(self.correction_name, (self.E,), init="bias"))
        for j, (u, d) in enumerate(zip(self.up_names, self.down_names)):
            if self.glu is not None:
                specs.append(TensorSpec(self.gate_names[j], (self.F, self.hidden)))
            specs += [TensorSpec(u, (self.F, self.hidden)), TensorSpec(d, (self.hidden, self.F))]
        if self.shared is not None:
            specs += self.shared.tensor_specs()
        return specs

    def elements_read_per_step(self) -> int:
        """A decode step reads the router and, per token, `top` experts: counted once (one token)."""
        own = self.shared.elements_read_per_step() if self.shared is not None else 0
        return own + self.E * self.hidden + self.E + self.top * (3 if self.glu is not None else 2) * self.F * self.hidden

    def bind(self, tensors, dtype, device):
        self.router.bind(tensors, dtype, device)
        if self.shared is not None:
            self.shared.bind(tensors, dtype, device)
        self.correction = tensors[self.correction_name].float().contiguous() if self.correction_name is not None else None
        self.tiled = False
        if self.glu is not None:                                                         # [E, 2 F, hidden]: gate rows, up rows
            self.tiled = dtype == torch.bfloat16 and self.hidden % 8 == 0 and self.F % 8 == 0
            if self.tiled:                                                               # 8 gate rows, their 8 up rows, and so on
                self.w_up = torch.stack([torch.stack([tensors[g].view(self.F // 8, 8, self.hidden), tensors[u].view(self.F // 8, 8, self.hidden)],
                                                     dim=1).reshape(2 * self.F, self.hidden)
                                         for g, u in zip(self.gate_names, self.up_names)]).contiguous()
            else:
                self.w_up = torch.stack([torch.cat([tensors[g], tensors[u]]) for g, u in zip(self.gate_names, self.up_names)]).contiguous()
        else:
            self.w_up = torch.stack([tensors[n] for n in self.up_names]).contiguous()    # [E, F, hidden]
        self.w_down = torch.stack([tensors[n] for n in self.down_names]).contiguous()    # [E, hidden, F]
        self.counts = torch.zeros((self.E,), dtype=torch.int32, device=device)
        if self.w_up.dtype != dtype:
            raise ValueError(f"the experts' matrices are {self.w_up.dtype}, the engine runs in {dtype}")

    def _on_tensor_cores(self, x) -> bool:
        """The grouped products can run on the tensor-core kernel: bfloat16, and the contraction widths (hidden for the
        experts' first product, their own width for the second) multiples of 8 elements (16 bytes for its copies)."""
        return x.dtype == torch.bfloat16 and self.hidden % 8 == 0 and self.F % 8 == 0 and x.data_ptr() % 16 == 0

    def forward(self, x, ctx):
        routed = self._routed(x, ctx)
        if self.shared is None:
            return routed
        return [routed, self.shared.forward(x, ctx)]

    def _routed(self, x, ctx):
        k = ctx.kernels.mix
        T, dev = x.shape[0], x.device
        pairs = T * self.top
        idx = torch.empty((T, self.top), dtype=torch.int32, device=dev)
        wgt = torch.empty((T, self.top), dtype=torch.float32, device=dev)
        z = self.router.forward(x, ctx, out_dtype=torch.float32)                  # logits, float32 sums
        k.moe_route(z, self.correction, idx, wgt, self.n_groups, self.keep, self.top, self.scale, router=self.router_kind)
        if pairs <= self.PAIRS_ONE_BY_ONE:
            hid = torch.empty((pairs, self.F), dtype=x.dtype, device=dev)
            out = torch.empty((self.top, T, self.hidden), dtype=torch.float32, device=dev)
            k.moe_pairs(x, self.w_up, self.w_down, idx, wgt, hid, out, glu=self.glu, tiled=self.tiled)
            return out
        offsets = torch.empty((self.E + 1,), dtype=torch.int32, device=dev)
        if not self._on_tensor_cores(x):
            pair_of_row = torch.empty((pairs,), dtype=torch.int32, device=dev)
            k.moe_group_rows(idx, self.counts, offsets, pair_of_row)
            hid = torch.empty((pairs, self.F), dtype=x.dtype, device=dev)
            out = torch.empty((self.top, T, self.hidden), dtype=torch.float32, device=dev)
            raw = torch.empty((pairs, 2 * self.F), dtype=x.dtype, device=dev) if self.glu is not None else None
            k.moe_grouped(x, self.w_up, self.w_down, wgt, offsets, pair_of_row, hid, out, glu=self.glu, raw=raw, tiled=self.tiled)
            return out
        # every expert's rows from a multiple of 128 on, so that a tile of the tensor-core product has one expert
        tile = 128
        rows = -(-(pairs + self.E * (tile - 1)) // tile) * tile
        pair_of_row = torch.empty((rows,), dtype=torch.int32, device=dev)
        row_of_pair = torch.empty((pairs,), dtype=torch.int32, device=dev)
        tile_group = torch.empty((rows // tile,), dtype=torch.int32, device=dev)
        k.moe_group_rows(idx, self.counts, offsets, pair_of_row, row_of_pair, tile_group, pad=tile)
        xs = torch.empty((rows, self.hidden), dtype=x.dtype, device=dev)
        k.moe_gather_rows(x, pair_of_row, self.top, xs)
        tc = ctx.kernels.tensor_core
        hid = torch.empty((rows, self.F), dtype=x.dtype, device=dev)
        if self.glu is not None:      # `tiled` holds here: its conditions are those of the tensor-core path
            tc.gemm_grouped(xs, self.w_up, hid, tile_group, ctx.err_flag, rows_used=offsets[self.E:], glu=self.glu)
        else:
            tc.gemm_grouped(xs, self.w_up, hid, tile_group, ctx.err_flag, act="relu_squared", rows_used=offsets[self.E:])
        ys = torch.empty((rows, self.hidden), dtype=torch.float32, device=dev)
        tc.gemm_grouped(hid, self.w_down, ys, tile_group, ctx.err_flag, rows_used=offsets[self.E:])
        out = torch.empty((T, self.hidden), dtype=torch.float32, device=dev)
        k.moe_combine(ys, row_of_pair, wgt, out)
        return out


FEED_FORWARDS.register("act_feed_forward", ActFeedForward)
FEED_FORWARDS.register("routed_experts", RoutedExperts)

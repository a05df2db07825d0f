"""Layout of the Tufazen decoder: which parts, with which numbers and tensor names.

The embedding is x = `embed`[token] + `bigram`[r], r a hash of (previous token, token) and the table's last row for a
sequence's first token. The two sublayers of a layer work side by side on the same normed stream: h = norm1(x) is formed
once, by a norm of the kind without statistics (tanh(alpha v) w + b; tensors `l<i>.norm1`, `.norm1.b`, `.norm1.alpha`), and
x += mixer(h) + ff(h).
Behind them the layer takes an input from the token itself, x += rms(P (gelu(G x) * e_token)) w (`l<i>.side.gate`,
`.side.proj`, `.side.norm`; the table `side.embed` is one tensor of which layer i reads its own columns, whichever pass
it runs in). A run of layers may be gone through several times with the same weights (`loop`): every appearance has a
cache unit of its own, and before pass t's first layer the stream takes the vector `loop.step`[t].

The mixer (`l<i>.mix.*`) is one of two. `attention`: grouped-query softmax attention without a value projection (the values
are the keys before the rotation), neighbouring pairs of the leading dims turned with frequencies rescaled along a ramp,
scores capped by tanh, a stored sink per head in the softmax's denominator (`sink`), and the concatenated heads multiplied
element by element with sigmoid(`g` h). `latent_attention`: queries through a normed latent (`dq`, `dq.norm`, `uq`), keys and
values from a cached normed latent (`dkv`, `dkv.norm`, `uk`, `uv`) with one rotated key part for all heads (dim i turned with
dim i + rot / 2), and a sigmoid gate per head (`g`).

The feed-forward (`l<i>.mlp.*`) is dense with the clamped gate g * sigmoid(1.702 g) * (u + 1) (`gate`, `up`, `down`), or
routed: softmax scores over all experts, groups rated by their best member, the best open experts weighted by their
scores as they are (`router`, `e<j>.gate|up|down`, silu-gated), beside a shared expert of the same form (`shared.*`).

The model's last norm `final.norm` is of the same kind; the head `head` is a matrix of its own and the logits are
multiplied by `logit_scale`.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.tufazen import TufazenAttentionConfig, TufazenConfig, TufazenDenseConfig
from ..engine.layout import ModelLayout, looped_schedule, sequential_schedule
from ..parts.base import PartSpec
from ..parts.block import LayerSpec
from ..parts.embedding import linear_head, token_embedding
from ..parts.rotary import YarnScaling

MAX_POSITIONS = 1 << 20      # the family states no longest sequence; the cache's size bounds it
GATE_SLOPE = 1.702           # the family's constant inside the dense feed-forward's sigmoid


def _norm(cfg: TufazenConfig, name: str) -> PartSpec:
    return PartSpec("dynamic_tanh", dict(width=cfg.width, weight_name=name, bias_name=name + ".b", alpha_name=name + ".alpha"))


def _rotary(rot, width: int, pairing: str) -> PartSpec | None:
    if rot is None:
        return None
    s = rot.scaling
    scaling = YarnScaling(s["factor"], s["original"], s["fast"], s["slow"]) if s is not None else None
    return PartSpec("rotary", dict(head_dim=width, rotary_dim=rot.dims, theta=rot.base, scaling=scaling, pairing=pairing))


def _mixer(cfg: TufazenConfig, layer, p: str) -> PartSpec:
    m = layer.mixer
    if isinstance(m, TufazenAttentionConfig):
        return PartSpec("attention", dict(
            hidden=cfg.width, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim, position=_rotary(m.rot, m.dim, "interleaved"),
            scale=m.scale, values_are_keys=True, softcap=m.softcap, sink_name=p + "sink", gate_name=p + "g", gate_per="element",
            q_name=p + "q", k_name=p + "k", v_name=None, o_name=p + "o"))
    return PartSpec("latent_attention", dict(
        hidden=cfg.width, n_heads=m.heads, dim=m.dim, rot_dim=m.rot_dim, v_dim=m.vdim, kv_rank=m.kv_rank, scale=m.scale,
        position=_rotary(m.rot, m.rot_dim, "half"), norm_eps=cfg.norm_eps, q_name=None, q_rank=m.q_rank, dq_name=p + "dq",
        dq_norm_name=p + "dq.norm", uq_name=p + "uq", uk_name=p + "uk", uv_name=p + "uv", o_name=p + "o", dkv_name=p + "dkv",
        dkv_norm_name=p + "dkv.norm", gate_name=p + "g", prompt_kernel="tensor"))


def _feed_forward(cfg: TufazenConfig, f, p: str) -> PartSpec:
    if isinstance(f, TufazenDenseConfig):
        return PartSpec("clamped_glu", dict(hidden=cfg.width, intermediate=f.ff, gate_name=p + "gate", up_name=p + "up",
                                            down_name=p + "down", limit=f.limit, alpha=GATE_SLOPE))
    names = lambda what: [f"{p}e{j}.{what}" for j in range(f.experts)]
    shared = None
    if f.shared_ff is not None:
        shared = PartSpec("swiglu", dict(hidden=cfg.width, intermediate=f.shared_ff, gate_name=p + "shared.gate",
                                         up_name=p + "shared.up", down_name=p + "shared.down"))
    return PartSpec("routed_experts", dict(
        hidden=cfg.width, intermediate=f.ff, experts=f.experts, top=f.top, n_groups=f.groups, keep_groups=f.keep, scale=1.0,
        router="grouped_softmax", router_name=p + "router", correction_name=None, act="silu_glu", gate_names=names("gate"),
        up_names=names("up"), down_names=names("down"), shared=shared))


def tufazen_layout(cfg: TufazenConfig) -> ModelLayout:
    layers = []
    n = len(cfg.layers)
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        parts = {"mixer_norm": _norm(cfg, p + "norm1"), "mixer": _mixer(cfg, layer, p + "mix.")}
        if layer.mlp is not None:
            parts["feed_forward"] = _feed_forward(cfg, layer.mlp, p + "mlp.")
        if cfg.side_dim is not None:
            parts["stream_input"] = PartSpec("token_side", dict(
                width=cfg.width, dim=cfg.side_dim, vocab=cfg.vocab, table_name="side.embed", table_width=n * cfg.side_dim,
                column=i * cfg.side_dim, gate_name=p + "side.gate", proj_name=p + "side.proj", norm_name=p + "side.norm",
                eps=cfg.norm_eps, owns_table=i == 0))
        layers.append(LayerSpec("parallel_input", parts))
    stream_parts: tuple[PartSpec, ...] = ()
    if cfg.loop is None:
        schedule = sequential_schedule(n)
    else:
        lp = cfg.loop
        stream_parts = tuple(PartSpec("pass_vector", dict(width=cfg.width, table_name="loop.step", rows=lp.times, row=t, owns_table=t == 0))
                             for t in range(lp.times))
        schedule = looped_schedule(n, lp.start, lp.stop, lp.times, before_pass=lambda t: (t,))
    if cfg.bigram is None:
        embedding = token_embedding(cfg.vocab, cfg.width, "embed")
    else:
        b = cfg.bigram
        embedding = PartSpec("pair_hash_embedding", dict(vocab=cfg.vocab, width=cfg.width, name="embed", pair_name="bigram",
                                                         buckets=b.buckets, mul_prev=b.mul_prev, mul_cur=b.mul_cur))
    return ModelLayout(
        vocab_size=cfg.vocab, hidden_size=cfg.width, max_positions=MAX_POSITIONS, embedding=embedding, layers=tuple(layers),
        schedule=schedule, final_norm=_norm(cfg, "final.norm"), head=linear_head(cfg.vocab, cfg.width, "head", scale=cfg.logit_scale),
        stream_parts=stream_parts)


register_architecture("Tufazen", TufazenConfig, tufazen_layout)

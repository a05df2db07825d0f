"""Layout of the Belasun decoder: which parts, with which numbers and tensor names.

A layer is x += mixer(norm1(x)); x += experts(norm2(x)) where it has a feed-forward; and, where the
model has a token-side table, x += rms(P (gelu(G x) * e_token)) w: an input from the token itself,
gated by the stream (`l<i>.side.gate`, `.side.proj`, `.side.norm`; the table `side.embed` is one
tensor of which layer i reads its own columns). The norms are RMS norms with plain weights
(`l<i>.norm1`, `.norm2`, `final.norm`).

The mixer (`l<i>.mix.*`) is grouped-query softmax attention with four additions: a short causal
convolution over time behind each of the three projections (`q.conv`, `k.conv`, `v.conv`), an RMS
norm over the whole query projection and over the whole key projection (`q.norm`, `k.norm`), a
rotation of the leading dims of every head in half pairing with the three-band rescaling of
frequencies by wavelength, and a sigmoid gate per head computed from the mixer's own input (`g`).
A query sees the earlier keys of its own chunk of positions only.

The feed-forward (`l<i>.mlp.*`) is routed experts: router logits with a bias (`router`, `router.b`),
the `top` largest picked and weighted by the softmax over the picked ones; an expert (`e<j>.gate`,
`.up`, `.down`) applies the clamped gate g * sigmoid(1.702 g) * (u + 1).

The embedding `embed` is also the output head, behind `final.norm`; the logits are capped by
cap * tanh(logits / cap) where the configuration gives a cap.
"""
from __future__ import annotations

from ..config.belasun import BelasunConfig
from ..config.registry import register_architecture
from ..engine.layout import ModelLayout, sequential_schedule
from ..parts.base import PartSpec
from ..parts.block import LayerSpec
from ..parts.embedding import linear_head, token_embedding

MAX_POSITIONS = 1 << 20      # the family states no longest sequence; the cache's size bounds it
GATE_SLOPE = 1.702           # the family's constant inside an expert's sigmoid


def _norm(cfg: BelasunConfig, name: str) -> PartSpec:
    return PartSpec("rmsnorm", dict(width=cfg.width, eps=cfg.norm_eps, weight_name=name))


def _mixer(cfg: BelasunConfig, layer, p: str) -> PartSpec:
    m = layer.mixer
    position = None
    if m.rot is not None:
        position = PartSpec("rotary", dict(head_dim=m.dim, rotary_dim=m.rot.dims, theta=m.rot.base, scaling=m.rot.scaling,
                                           pairing="half"))
    conv = dict(taps=m.conv, q_name=p + "q.conv", k_name=p + "k.conv", v_name=p + "v.conv") if m.conv > 1 else None
    return PartSpec("attention", dict(
        hidden=cfg.width, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim, v_dim=m.vdim, position=position,
        scale=m.scale, chunk=m.chunk, conv=conv, qk_norm=dict(q_name=p + "q.norm", k_name=p + "k.norm", eps=cfg.norm_eps),
        gate_name=p + "g", q_name=p + "q", k_name=p + "k", v_name=p + "v", o_name=p + "o"))


def _feed_forward(cfg: BelasunConfig, f, p: str) -> PartSpec:
    names = lambda what: [f"{p}e{j}.{what}" for j in range(f.experts)]
    return PartSpec("routed_experts", dict(
        hidden=cfg.width, intermediate=f.ff, experts=f.experts, top=f.top, n_groups=1, keep_groups=1, scale=1.0,
        router="top_softmax", router_name=p + "router", correction_name=p + "router.b", act="clamped_glu",
        gate_names=names("gate"), up_names=names("up"), down_names=names("down"), limit=f.limit, alpha=GATE_SLOPE))


def belasun_layout(cfg: BelasunConfig) -> ModelLayout:
    layers = []
    n = len(cfg.layers)
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        parts = {"mixer_norm": _norm(cfg, p + "norm1"), "mixer": _mixer(cfg, layer, p + "mix.")}
        if layer.mlp is not None:
            parts.update(feed_forward_norm=_norm(cfg, p + "norm2"), feed_forward=_feed_forward(cfg, layer.mlp, p + "mlp."))
        if cfg.side_dim is not None:
            parts["stream_input"] = PartSpec("token_side", dict(
                width=cfg.width, dim=cfg.side_dim, vocab=cfg.vocab, table_name="side.embed", table_width=n * cfg.side_dim,
                column=i * cfg.side_dim, gate_name=p + "side.gate", proj_name=p + "side.proj", norm_name=p + "side.norm",
                eps=cfg.norm_eps, owns_table=i == 0))
        layers.append(LayerSpec("pre_norm_input", parts))
    return ModelLayout(
        vocab_size=cfg.vocab, hidden_size=cfg.width, max_positions=MAX_POSITIONS,
        embedding=token_embedding(cfg.vocab, cfg.width, "embed"), layers=tuple(layers), schedule=sequential_schedule(n),
        final_norm=_norm(cfg, "final.norm"), head=linear_head(cfg.vocab, cfg.width, "embed", tied=True, softcap=cfg.logit_softcap))


register_architecture("Belasun", BelasunConfig, belasun_layout)

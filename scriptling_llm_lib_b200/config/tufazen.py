"""TufazenConfig: the sizes, constants and order of layers of a Tufazen decoder, from config.json.

The file is nested like the other in-house families': `layers` lists the layers, each with its `type` (the mixer:
`attention`, grouped-query attention whose values are its keys, or `latent_attention`, attention over a cached latent),
the mixer's sizes and constants under `mixer`, and its feed-forward under `mlp` (null: none; `kind` dense or moe).
Model-wide: `vocab`, `width`, `norm.eps`, `logit_scale` (absent: 1), `embedding.bigram` (`buckets`, `mul_prev`,
`mul_cur`; absent: a plain embedding), `token_side.dim` (absent: the layers take no input from the token itself) and
`loop` (`start`, `stop`, `times`: the model goes through the run of layers from `start` up to, not including, `stop`
that many times on one set of weights before it goes on; absent: every layer once). Every layer states its own sizes, so two layers of a model may differ in all of them.

An `attention` mixer: `heads`, `kv_heads`, `dim` (query/key width of a head), `vdim` (value width; the values are the
keys, so it equals `dim`), `scale` (multiplies q . k), `softcap` (absent: scores as they are), `rot` (`dims` leading dims
of a head that turn in neighbouring pairs, `base`, optionally `scaling` with `factor`, `original`, `fast`, `slow`; no
`rot`: no rotation). A `latent_attention` mixer: `heads`, `dim` and `rot_dim` (unrotated and rotated query/key dims of a
head), `vdim`, `kv_rank`, `q_rank`, `scale`, `rot` (`base`, `dims` = `rot_dim`; dim i turns with dim i + dims / 2).
A dense feed-forward: `ff`, `limit`. A routed one: `expert.ff`, `router.experts`, `router.top`, `router.groups`
(`count`, `keep`; absent: one group) and `shared.ff` (absent: no shared expert).
"""
from __future__ import annotations

from dataclasses import dataclass, field

from .base import ConfigError, KeyReader

LAYER_TYPES = ("attention", "latent_attention")


@dataclass(frozen=True)
class TufazenRotation:
    dims: int
    base: float
    scaling: dict | None       # {"factor", "original", "fast", "slow"} or None


@dataclass(frozen=True)
class TufazenAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float | None
    rot: TufazenRotation | None


@dataclass(frozen=True)
class TufazenLatentConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot: TufazenRotation | None


@dataclass(frozen=True)
class TufazenDenseConfig:
    ff: int
    limit: float


@dataclass(frozen=True)
class TufazenMoeConfig:
    ff: int
    experts: int
    top: int
    groups: int
    keep: int
    shared_ff: int | None


@dataclass(frozen=True)
class TufazenLayerConfig:
    type: str
    mixer: TufazenAttentionConfig | TufazenLatentConfig
    mlp: TufazenDenseConfig | TufazenMoeConfig | None


@dataclass(frozen=True)
class TufazenBigram:
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class TufazenLoop:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class TufazenConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    logit_scale: float
    bigram: TufazenBigram | None
    side_dim: int | None
    loop: TufazenLoop | None
    layers: tuple[TufazenLayerConfig, ...]
    raw: dict = field(default_factory=dict, compare=False, repr=False)

    def to_json_dict(self) -> dict:
        """The config.json that reads back as this record."""
        def rot(r: TufazenRotation | None):
            if r is None:
                return None
            out = {"base": r.base, "dims": r.dims}
            if r.scaling is not None:
                out["scaling"] = dict(r.scaling)
            return out

        def mixer(m):
            if isinstance(m, TufazenAttentionConfig):
                out = {"dim": m.dim, "heads": m.heads, "kv_heads": m.kv_heads, "scale": m.scale, "vdim": m.vdim}
                if m.softcap is not None:
                    out["softcap"] = m.softcap
            else:
                out = {"dim": m.dim, "heads": m.heads, "kv_rank": m.kv_rank, "q_rank": m.q_rank, "rot_dim": m.rot_dim,
                       "scale": m.scale, "vdim": m.vdim}
            if m.rot is not None:
                out["rot"] = rot(m.rot)
            return out

        def mlp(f):
            if f is None:
                return None
            if isinstance(f, TufazenDenseConfig):
                return {"ff": f.ff, "kind": "dense", "limit": f.limit}
            out = {"expert": {"ff": f.ff}, "kind": "moe",
                   "router": {"experts": f.experts, "groups": {"count": f.groups, "keep": f.keep}, "top": f.top}}
            if f.shared_ff is not None:
                out["shared"] = {"ff": f.shared_ff}
            return out
        out = {"architecture": self.architecture,
               "layers": [{"mixer": mixer(l.mixer), "mlp": mlp(l.mlp), "type": l.type} for l in self.layers],
               "logit_scale": self.logit_scale, "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.bigram is not None:
            out["embedding"] = {"bigram": {"buckets": self.bigram.buckets, "mul_cur": self.bigram.mul_cur,
                                           "mul_prev": self.bigram.mul_prev}}
        if self.side_dim is not None:
            out["token_side"] = {"dim": self.side_dim}
        if self.loop is not None:
            out["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        return out

    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json") -> "TufazenConfig":
        r = KeyReader(raw, where)
        name = r.string("architecture", default=None)
        if name is None:
            archs = r.any("architectures")
            if not (isinstance(archs, list) and archs and isinstance(archs[0], str)):
                raise ConfigError(f"{where}: 'architecture' must name the model")
            name = archs[0]
        vocab = r.integer("vocab", minimum=1)
        width = r.integer("width", minimum=1)
        eps = KeyReader(_obj(r, "norm", where), where + ":norm").number("eps", positive=True)
        logit_scale = r.number("logit_scale", default=1.0)
        bigram = None
        emb = r.any("embedding")
        if emb is not None:
            e = KeyReader(_obj(r, "embedding", where), where + ":embedding")
            if e.any("bigram") is not None:
                b = KeyReader(_obj(e, "bigram", where + ":embedding"), where + ":embedding:bigram")
                bigram = TufazenBigram(b.integer("buckets", minimum=1), b.integer("mul_prev", minimum=0), b.integer("mul_cur", minimum=0))
        side_dim = None
        if r.any("token_side") is not None:
            side_dim = KeyReader(_obj(r, "token_side", where), where + ":token_side").integer("dim", minimum=1)
        entries = r.any("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError(f"{where}: 'layers' must be a list with an entry per layer")
        layers = tuple(_layer(e, f"{where}:layers[{i}]") for i, e in enumerate(entries))
        loop = None
        if r.any("loop") is not None:
            lw = where + ":loop"
            lo = KeyReader(_obj(r, "loop", where), lw)
            loop = TufazenLoop(lo.integer("start", minimum=0), lo.integer("stop", minimum=0), lo.integer("times", minimum=1))
            if not loop.start < loop.stop <= len(layers):
                raise ConfigError(f"{lw}: layers {loop.start} .. {loop.stop - 1} are not a run of the model's {len(layers)} layers")
        return cls(name, vocab, width, eps, logit_scale, bigram, side_dim, loop, layers, raw)


def _obj(r: KeyReader, key: str, where: str) -> dict:
    v = r.any(key)
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: {key!r} must be an object")
    return v


def _rotation(m: KeyReader, mw: str, width: int, scaled: bool) -> TufazenRotation | None:
    if m.any("rot") is None:
        return None
    rw = mw + ":rot"
    rot = KeyReader(_obj(m, "rot", mw), rw)
    dims = rot.integer("dims", minimum=0)
    if dims % 2 or dims > width:
        raise ConfigError(f"{rw}: 'dims' ({dims}) must be even and at most the rotated width ({width})")
    if dims < 2:
        return None
    scaling = rot.any("scaling")
    if scaling is not None:
        s = KeyReader(scaling, rw + ":scaling")
        scaling = {"factor": s.number("factor", positive=True), "original": s.number("original", positive=True),
                   "fast": s.number("fast", positive=True), "slow": s.number("slow", positive=True)}
    base = rot.number("base", positive=True)
    if scaling is not None and not base > 1:
        raise ConfigError(f"{rw}: a rescaled rotation needs a base above 1")
    return TufazenRotation(dims, base, scaling)


def _layer(e, where: str) -> TufazenLayerConfig:
    r = KeyReader(e, where)
    kind = r.string("type", choices=LAYER_TYPES)
    mw = where + ":mixer"
    m = KeyReader(_obj(r, "mixer", where), mw)
    heads, dim, vdim = m.integer("heads", minimum=1), m.integer("dim", minimum=1), m.integer("vdim", minimum=1)
    if kind == "attention":
        kv_heads = m.integer("kv_heads", minimum=1)
        if heads % kv_heads:
            raise ConfigError(f"{mw}: 'kv_heads' ({kv_heads}) must divide 'heads' ({heads})")
        if vdim != dim:
            raise ConfigError(f"{mw}: the values are the keys, so 'vdim' ({vdim}) must equal 'dim' ({dim})")
        mixer = TufazenAttentionConfig(heads, kv_heads, dim, vdim, m.number("scale"), m.number("softcap", default=None, positive=True),
                                       _rotation(m, mw, dim, True))
    else:
        rot_dim = m.integer("rot_dim", minimum=0)
        rot = _rotation(m, mw, rot_dim, False)
        mixer = TufazenLatentConfig(heads, dim, rot_dim, vdim, m.integer("kv_rank", minimum=1), m.integer("q_rank", minimum=1),
                                    m.number("scale"), rot)
    mlp = r.any("mlp")
    ff = None
    if mlp is not None:
        fw = where + ":mlp"
        f = KeyReader(mlp, fw)
        if f.string("kind", choices=("dense", "moe")) == "dense":
            ff = TufazenDenseConfig(f.integer("ff", minimum=1), f.number("limit", positive=True))
        else:
            ex = KeyReader(_obj(f, "expert", fw), fw + ":expert")
            ro = KeyReader(_obj(f, "router", fw), fw + ":router")
            experts, top = ro.integer("experts", minimum=1), ro.integer("top", minimum=1)
            groups, keep = 1, 1
            if ro.any("groups") is not None:
                g = KeyReader(_obj(ro, "groups", fw + ":router"), fw + ":router:groups")
                groups, keep = g.integer("count", minimum=1), g.integer("keep", minimum=1)
            if experts % groups or keep > groups or top > keep * (experts // groups):
                raise ConfigError(f"{fw}:router: {experts} experts in {groups} groups of which {keep} stay open cannot give "
                                  f"{top} to a token")
            shared = None
            if f.any("shared") is not None:
                shared = KeyReader(_obj(f, "shared", fw), fw + ":shared").integer("ff", minimum=1)
            ff = TufazenMoeConfig(ex.integer("ff", minimum=1), experts, top, groups, keep, shared)
    return TufazenLayerConfig(kind, mixer, ff)

"""BelasunConfig: the sizes, constants and order of layers of a Belasun decoder, from config.json.

The file is nested like the other in-house families': `layers` lists the layers, each with its
`type` (the mixer; this family has one, `attention`), the mixer's sizes and constants under `mixer`
and its feed-forward under `mlp` (null: none; `kind` moe). Model-wide: `vocab`, `width`,
`norm.eps`, `logit_softcap` (absent or null: the logits leave as they are) and `token_side.dim`
(absent or null: the layers take no input from the token itself). Every layer states its own
sizes, so two layers of a model may differ in all of them.

A mixer: `heads`, `kv_heads`, `dim` (query/key width of a head), `vdim` (value width), `scale`
(multiplies q . k), `conv` (taps of the short convolution behind the projections; absent or 1:
none), `mask.size` (positions per chunk; no `mask`: every earlier key is seen), `rot` (`dims`
leading dims of a head that turn, `base`, and optionally `scaling` with `factor`, `low`, `high`,
`original`; no `rot` or `dims` 0: no rotation).
"""
from __future__ import annotations

from dataclasses import dataclass, field

from .base import ConfigError, KeyReader
from .llama import RopeScaling

LAYER_TYPES = ("attention",)


@dataclass(frozen=True)
class BelasunRotation:
    dims: int                      # leading dims of every head that turn, dim i with dim i + dims / 2
    base: float
    scaling: RopeScaling | None    # the three-band rescaling by wavelength ("llama3") or None


@dataclass(frozen=True)
class BelasunAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    conv: int                      # taps; 1: no convolution
    chunk: int | None              # positions per chunk; None: no chunks
    rot: BelasunRotation | None


@dataclass(frozen=True)
class BelasunMoeConfig:
    ff: int
    limit: float
    experts: int
    top: int


@dataclass(frozen=True)
class BelasunLayerConfig:
    type: str
    mixer: BelasunAttentionConfig
    mlp: BelasunMoeConfig | None


@dataclass(frozen=True)
class BelasunConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    logit_softcap: float | None
    side_dim: int | None
    layers: tuple[BelasunLayerConfig, ...]
    raw: dict = field(default_factory=dict, compare=False, repr=False)

    def to_json_dict(self) -> dict:
        """The config.json that reads back as this record."""
        def mixer(m: BelasunAttentionConfig):
            out = {"conv": m.conv, "dim": m.dim, "heads": m.heads, "kv_heads": m.kv_heads, "scale": m.scale, "vdim": m.vdim}
            if m.chunk is not None:
                out["mask"] = {"size": m.chunk}
            if m.rot is not None:
                rot = {"base": m.rot.base, "dims": m.rot.dims}
                s = m.rot.scaling
                if s is not None:
                    rot["scaling"] = {"factor": s.factor, "high": s.high_freq_factor, "low": s.low_freq_factor,
                                      "original": s.original_max_position_embeddings}
                out["rot"] = rot
            return out

        def mlp(f: BelasunMoeConfig | None):
            if f is None:
                return None
            return {"expert": {"ff": f.ff, "limit": f.limit}, "kind": "moe", "router": {"experts": f.experts, "top": f.top}}
        out = {"architecture": self.architecture,
               "layers": [{"mixer": mixer(l.mixer), "mlp": mlp(l.mlp), "type": l.type} for l in self.layers],
               "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        if self.side_dim is not None:
            out["token_side"] = {"dim": self.side_dim}
        return out

    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json") -> "BelasunConfig":
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
        cap = r.number("logit_softcap", default=None, positive=True)
        side = r.any("token_side")
        side_dim = None
        if side is not None:
            side_dim = KeyReader(_obj(r, "token_side", where), where + ":token_side").integer("dim", minimum=1)
        entries = r.any("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError(f"{where}: 'layers' must be a list with an entry per layer")
        layers = tuple(_layer(e, f"{where}:layers[{i}]") for i, e in enumerate(entries))
        return cls(name, vocab, width, eps, cap, side_dim, layers, raw)


def _obj(r: KeyReader, key: str, where: str) -> dict:
    v = r.any(key)
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: {key!r} must be an object")
    return v


def _layer(e, where: str) -> BelasunLayerConfig:
    r = KeyReader(e, where)
    kind = r.string("type", choices=LAYER_TYPES)
    mw = where + ":mixer"
    m = KeyReader(_obj(r, "mixer", where), mw)
    heads, kv_heads = m.integer("heads", minimum=1), m.integer("kv_heads", minimum=1)
    if heads % kv_heads:
        raise ConfigError(f"{mw}: {heads} heads cannot share {kv_heads} key/value heads")
    dim = m.integer("dim", minimum=1)
    chunk = None
    if m.any("mask") is not None:
        chunk = KeyReader(_obj(m, "mask", mw), mw + ":mask").integer("size", minimum=1)
    rotation = None
    if m.any("rot") is not None:
        rw = mw + ":rot"
        rot = KeyReader(_obj(m, "rot", mw), rw)
        dims = rot.integer("dims", minimum=0)
        if dims % 2 or dims > dim:
            raise ConfigError(f"{rw}: 'dims' ({dims}) must be even and at most the head's width ({dim})")
        scaling = rot.any("scaling")
        if scaling is not None:
            s = KeyReader(scaling, rw + ":scaling")
            scaling = RopeScaling("llama3", s.number("factor", positive=True), s.number("low", positive=True),
                                  s.number("high", positive=True), s.number("original", positive=True))
            if scaling.high_freq_factor == scaling.low_freq_factor:
                raise ConfigError(f"{rw}:scaling: 'high' and 'low' must differ")
        if dims >= 2:
            rotation = BelasunRotation(dims, rot.number("base", positive=True), scaling)
    mixer = BelasunAttentionConfig(heads, kv_heads, dim, m.integer("vdim", minimum=1), m.number("scale"),
                                   m.integer("conv", default=1, minimum=1), chunk, rotation)
    mlp = r.any("mlp")
    ff = None
    if mlp is not None:
        fw = where + ":mlp"
        f = KeyReader(mlp, fw)
        f.string("kind", choices=("moe",))
        ex = KeyReader(_obj(f, "expert", fw), fw + ":expert")
        ro = KeyReader(_obj(f, "router", fw), fw + ":router")
        ff = BelasunMoeConfig(ex.integer("ff", minimum=1), ex.number("limit", positive=True), ro.integer("experts", minimum=1),
                              ro.integer("top", minimum=1))
        if ff.top > ff.experts:
            raise ConfigError(f"{fw}:router: {ff.experts} experts cannot give {ff.top} to a token")
    return BelasunLayerConfig(kind, mixer, ff)

"""Typed configuration of the Zoporax decoder, read from its config.json keys.

A Zoporax model is a list of layers; each layer names its mixer (`type`: "latent_attention" or
"lightning"), gives the mixer's sizes and constants (`mixer`) and its feed-forward (`mlp`, or null
for a layer without one).  Every size and constant is per layer.

    architecture   "Zoporax"
    vocab, width   vocabulary and residual width (the output head reads the embedding table)
    norm.eps       epsilon of every RMS norm
    layers[i]      {"type", "mixer": {...}, "mlp": {...} | null}

latent_attention: `heads`, `dim` (unrotated query/key size of a head), `rot_dim` (rotated size), `vdim`,
`q_rank`, `kv_rank`, `scale`, `mask.size` (the window; absent: every earlier token), `rot` = {"dims", "base",
"scaling": {"factor", "original", "fast", "slow"} | absent}.
lightning: `heads`, `dim`, `vdim`, `decay` (one number per head).
mlp: {"kind": "dense", "ff"} (gated, with biases) or {"kind": "moe", "expert": {"ff"}, "router": {"experts",
"top", "scale", "groups": {"count", "keep"}}, "shared": {"ff"} | absent}.
"""
from __future__ import annotations

from dataclasses import dataclass

from .base import ConfigError, KeyReader, read_config_json

MIXERS = ("latent_attention", "lightning")


def _object(data, key: str, where: str, required: bool = True):
    value = data.get(key)
    if value is None:
        if required:
            raise ConfigError(f"{where}: required key '{key}' is missing")
        return None
    if not isinstance(value, dict):
        raise ConfigError(f"{where}: '{key}' must be an object, found {value!r}")
    return value


@dataclass(frozen=True)
class YarnRotation:
    dims: int
    base: float
    factor: float | None = None       # with a factor: original, fast and slow are given too
    original: float | None = None
    fast: float | None = None
    slow: float | None = None

    @classmethod
    def from_dict(cls, data, where: str, size: int) -> "YarnRotation | None":
        if data is None:
            return None
        r = KeyReader(data, f"{where}.rot")
        dims = r.integer("dims", size, minimum=0)
        if dims == 0:
            return None
        if dims % 2 or dims > size:
            raise ConfigError(f"{where}.rot: 'dims' {dims} must be even and at most the rotated size {size}")
        more = {}
        scaling = _object(data, "scaling", f"{where}.rot", required=False)
        if scaling is not None:
            s = KeyReader(scaling, f"{where}.rot.scaling")
            more = {k: s.number(k, positive=True) for k in ("factor", "original", "fast", "slow")}
        return cls(dims=dims, base=r.number("base", positive=True), **more)

    def to_dict(self) -> dict:
        out = {"dims": self.dims, "base": self.base}
        if self.factor is not None:
            out["scaling"] = {"factor": self.factor, "original": self.original, "fast": self.fast, "slow": self.slow}
        return out


@dataclass(frozen=True)
class RouterConfig:
    experts: int
    top: int
    scale: float = 1.0
    groups: int = 1
    keep: int = 1


@dataclass(frozen=True)
class ZoporaxFeedForward:
    kind: str                          # "dense" or "moe"
    ff: int                            # dense: the hidden size; moe: an expert's hidden size
    router: RouterConfig | None = None
    shared_ff: int | None = None

    @classmethod
    def from_dict(cls, data, where: str) -> "ZoporaxFeedForward | None":
        if data is None:
            return None
        if not isinstance(data, dict):
            raise ConfigError(f"{where}: 'mlp' must be an object or null")
        where = f"{where}.mlp"
        kind = KeyReader(data, where).string("kind", "dense")
        if kind == "dense":
            return cls(kind=kind, ff=KeyReader(data, where).integer("ff", minimum=1))
        if kind != "moe":
            raise ConfigError(f"{where}: kind {kind!r} is not supported (supported: 'dense', 'moe')")
        ff = KeyReader(_object(data, "expert", where), f"{where}.expert").integer("ff", minimum=1)
        rd = _object(data, "router", where)
        r = KeyReader(rd, f"{where}.router")
        experts, top = r.integer("experts", minimum=1), r.integer("top", minimum=1)
        gd = _object(rd, "groups", f"{where}.router", required=False)
        groups, keep = 1, 1
        if gd is not None:
            g = KeyReader(gd, f"{where}.router.groups")
            groups, keep = g.integer("count", minimum=1), g.integer("keep", minimum=1)
        if experts % groups or keep > groups:
            raise ConfigError(f"{where}.router: {experts} experts cannot form {groups} equal groups of which {keep} are kept")
        if top > keep * (experts // groups):
            raise ConfigError(f"{where}.router: 'top' {top} exceeds the {keep * (experts // groups)} experts of the kept groups")
        sd = _object(data, "shared", where, required=False)
        shared = KeyReader(sd, f"{where}.shared").integer("ff", minimum=1) if sd is not None else None
        return cls(kind=kind, ff=ff, router=RouterConfig(experts, top, r.number("scale", 1.0), groups, keep), shared_ff=shared)

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        r = self.router
        out = {"kind": "moe", "expert": {"ff": self.ff},
               "router": {"experts": r.experts, "top": r.top, "scale": r.scale, "groups": {"count": r.groups, "keep": r.keep}}}
        if self.shared_ff is not None:
            out["shared"] = {"ff": self.shared_ff}
        return out


@dataclass(frozen=True)
class ZoporaxLayer:
    type: str
    heads: int
    dim: int
    vdim: int
    mlp: ZoporaxFeedForward | None
    rot_dim: int | None = None               # latent_attention
    q_rank: int | None = None
    kv_rank: int | None = None
    scale: float | None = None
    window: int | None = None
    rot: YarnRotation | None = None
    decay: tuple[float, ...] | None = None   # lightning

    def to_dict(self) -> dict:
        m = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim}
        if self.type == "latent_attention":
            m.update(rot_dim=self.rot_dim, q_rank=self.q_rank, kv_rank=self.kv_rank, scale=self.scale)
            if self.window is not None:
                m["mask"] = {"size": self.window}
            if self.rot is not None:
                m["rot"] = self.rot.to_dict()
        else:
            m["decay"] = list(self.decay)
        return {"type": self.type, "mixer": m, "mlp": None if self.mlp is None else self.mlp.to_dict()}


def _layer(i: int, data) -> ZoporaxLayer:
    where = f"config.json: layers[{i}]"
    if not isinstance(data, dict):
        raise ConfigError(f"{where} must be an object")
    kind = KeyReader(data, where).string("type")
    if kind not in MIXERS:
        raise ConfigError(f"{where}: type {kind!r} is not one of {', '.join(MIXERS)}")
    mixer = _object(data, "mixer", where)
    m = KeyReader(mixer, f"{where}.mixer")
    heads, dim = m.integer("heads", minimum=1), m.integer("dim", minimum=1)
    vdim = m.integer("vdim", dim, minimum=1)
    mlp = ZoporaxFeedForward.from_dict(data.get("mlp"), where)
    more = {}
    if kind == "latent_attention":
        rot_dim = m.integer("rot_dim", minimum=0)
        more.update(rot_dim=rot_dim, q_rank=m.integer("q_rank", minimum=1), kv_rank=m.integer("kv_rank", minimum=1),
                    scale=m.number("scale", (dim + rot_dim) ** -0.5))
        mask = _object(mixer, "mask", f"{where}.mixer", required=False)
        if mask is not None:
            more["window"] = KeyReader(mask, f"{where}.mixer.mask").integer("size", None, minimum=1)
        rot = _object(mixer, "rot", f"{where}.mixer", required=False)
        more["rot"] = YarnRotation.from_dict(rot, f"{where}.mixer", rot_dim) if rot_dim else None
    else:
        decay = mixer.get("decay")
        if (not isinstance(decay, list) or len(decay) != heads
                or not all(isinstance(d, (int, float)) and not isinstance(d, bool) for d in decay)):
            raise ConfigError(f"{where}.mixer: 'decay' must list one number for each of the {heads} heads")
        more["decay"] = tuple(float(d) for d in decay)
    return ZoporaxLayer(type=kind, heads=heads, dim=dim, vdim=vdim, mlp=mlp, **more)


@dataclass(frozen=True)
class ZoporaxConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple[ZoporaxLayer, ...]
    max_positions: int = 32768           # no key of the design bounds a sequence; this sizes tables and default caches
    architectures: tuple[str, ...] = ("Zoporax",)

    @classmethod
    def from_dict(cls, data: dict) -> "ZoporaxConfig":
        r = KeyReader(data)
        norm = _object(data, "norm", "config.json")
        layers = data.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        return cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1),
                   norm_eps=KeyReader(norm, "config.json: norm").number("eps", positive=True),
                   layers=tuple(_layer(i, layer) for i, layer in enumerate(layers)),
                   max_positions=r.integer("max_positions", 32768, minimum=1))

    @classmethod
    def from_json(cls, folder_or_file) -> "ZoporaxConfig":
        return cls.from_dict(read_config_json(folder_or_file))

    def to_dict(self) -> dict:
        out = {"architecture": "Zoporax", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "layers": [layer.to_dict() for layer in self.layers]}
        if self.max_positions != 32768:
            out["max_positions"] = self.max_positions
        return out

"""Typed configuration of the Fetorax decoder, read from its config.json keys.

A Fetorax model is a list of layers; each layer names its mixer (`type`: "attention",
"retention" or "mlstm"), gives the mixer's sizes and constants (`mixer`) and its
feed-forward (`mlp`, or null for a layer without one).  Every size and constant is
per layer, so two layers of one model may differ in all of them.

    architecture   "Fetorax"
    vocab, width   vocabulary and residual width
    norm.eps       epsilon of every RMS norm (the layers' and the per-head unit norms)
    logit_softcap  c in logits <- c tanh(logits / c) (absent or null: no cap)
    layers[i]      {"type", "mixer": {...}, "mlp": {"kind": "dense", "ff": F} | null}

Mixer keys: `heads`, `dim` (query/key size of a head), `vdim` (value size); attention adds
`kv_heads`, `scale`, `rot`, and optionally `kv_from` (the layer whose keys and values it
reads); retention adds `decay` (one number per head) and `rot`; mlstm adds `gate_cap`.
`rot` = {"dims", "base", "scaling": {"factor"}} rotates the first `dims` dimensions of a
head, all frequencies divided by the factor.
"""
from __future__ import annotations

from dataclasses import dataclass

from .base import ConfigError, KeyReader, read_config_json

MIXERS = ("attention", "retention", "mlstm")


@dataclass(frozen=True)
class Rotation:
    dims: int
    base: float
    factor: float | None = None        # linear scaling: every frequency divided by it

    @classmethod
    def from_dict(cls, data, where: str, head_size: int) -> "Rotation | None":
        if data is None:
            return None
        if not isinstance(data, dict):
            raise ConfigError(f"{where}: 'rot' must be an object or null, found {data!r}")
        r = KeyReader(data, f"{where}.rot")
        dims = r.integer("dims", minimum=0)
        if dims == 0:
            return None
        if dims % 2 or dims > head_size:
            raise ConfigError(f"{where}.rot: 'dims' {dims} must be even and at most the head's size {head_size}")
        factor = None
        scaling = data.get("scaling")
        if scaling is not None:
            if not isinstance(scaling, dict):
                raise ConfigError(f"{where}.rot: 'scaling' must be an object or null, found {scaling!r}")
            factor = KeyReader(scaling, f"{where}.rot.scaling").number("factor", positive=True)
        return cls(dims=dims, base=r.number("base", positive=True), factor=factor)

    def to_dict(self) -> dict:
        out = {"dims": self.dims, "base": self.base}
        if self.factor is not None:
            out["scaling"] = {"factor": self.factor}
        return out


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str
    ff: int


@dataclass(frozen=True)
class FetoraxLayer:
    type: str
    heads: int
    dim: int
    vdim: int
    mlp: FeedForwardConfig | None
    kv_heads: int | None = None          # attention
    scale: float | None = None           # attention
    kv_from: int | None = None           # attention: the layer whose keys and values this one reads
    rot: Rotation | None = None          # attention, retention
    decay: tuple[float, ...] | None = None   # retention
    gate_cap: float | None = None        # mlstm

    def to_dict(self) -> dict:
        m = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim}
        if self.type == "attention":
            m.update(kv_heads=self.kv_heads, scale=self.scale)
            if self.kv_from is not None:
                m["kv_from"] = self.kv_from
        if self.type == "retention":
            m["decay"] = list(self.decay)
        if self.type == "mlstm":
            m["gate_cap"] = self.gate_cap
        if self.rot is not None:
            m["rot"] = self.rot.to_dict()
        return {"type": self.type, "mixer": m,
                "mlp": None if self.mlp is None else {"kind": self.mlp.kind, "ff": self.mlp.ff}}


def _layer(i: int, data) -> FetoraxLayer:
    where = f"config.json: layers[{i}]"
    if not isinstance(data, dict):
        raise ConfigError(f"{where} must be an object")
    kind = KeyReader(data, where).string("type")
    if kind not in MIXERS:
        raise ConfigError(f"{where}: type {kind!r} is not one of {', '.join(MIXERS)}")
    mixer = data.get("mixer")
    if not isinstance(mixer, dict):
        raise ConfigError(f"{where}: 'mixer' must be an object")
    m = KeyReader(mixer, f"{where}.mixer")
    heads, dim = m.integer("heads", minimum=1), m.integer("dim", minimum=1)
    vdim = m.integer("vdim", dim, minimum=1)
    mlp = data.get("mlp")
    if mlp is not None:
        if not isinstance(mlp, dict):
            raise ConfigError(f"{where}: 'mlp' must be an object or null")
        f = KeyReader(mlp, f"{where}.mlp")
        mlp = FeedForwardConfig(kind=f.string("kind", "dense"), ff=f.integer("ff", minimum=1))
        if mlp.kind != "dense":
            raise ConfigError(f"{where}.mlp: kind {mlp.kind!r} is not supported (supported: 'dense')")
    more = {}
    if kind == "attention":
        more["kv_heads"] = m.integer("kv_heads", heads, minimum=1)
        if heads % more["kv_heads"]:
            raise ConfigError(f"{where}.mixer: {heads} heads are not a multiple of {more['kv_heads']} kv_heads")
        more["scale"] = m.number("scale", dim ** -0.5)
        more["kv_from"] = m.integer("kv_from", None, minimum=0)
    if kind in ("attention", "retention"):
        more["rot"] = Rotation.from_dict(mixer.get("rot"), f"{where}.mixer", dim)
    if kind == "retention":
        decay = mixer.get("decay")
        if (not isinstance(decay, list) or len(decay) != heads
                or not all(isinstance(d, (int, float)) and not isinstance(d, bool) for d in decay)):
            raise ConfigError(f"{where}.mixer: 'decay' must list one number for each of the {heads} heads")
        more["decay"] = tuple(float(d) for d in decay)
    if kind == "mlstm":
        more["gate_cap"] = m.number("gate_cap", positive=True)
    return FetoraxLayer(type=kind, heads=heads, dim=dim, vdim=vdim, mlp=mlp, **more)


@dataclass(frozen=True)
class FetoraxConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple[FetoraxLayer, ...]
    logit_softcap: float | None = None
    max_positions: int = 32768           # no key of the design bounds a sequence; this sizes tables and default caches
    architectures: tuple[str, ...] = ("Fetorax",)

    @classmethod
    def from_dict(cls, data: dict) -> "FetoraxConfig":
        r = KeyReader(data)
        norm = data.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        layers = data.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        cfg = cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1),
                  norm_eps=KeyReader(norm, "config.json: norm").number("eps", positive=True),
                  layers=tuple(_layer(i, layer) for i, layer in enumerate(layers)),
                  logit_softcap=r.number("logit_softcap", None, positive=True),
                  max_positions=r.integer("max_positions", 32768, minimum=1))
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, folder_or_file) -> "FetoraxConfig":
        return cls.from_dict(read_config_json(folder_or_file))

    def validate(self) -> None:
        for i, layer in enumerate(self.layers):
            j = layer.kv_from
            if j is None:
                continue
            where = f"config.json: layers[{i}].mixer"
            if not 0 <= j < i:
                raise ConfigError(f"{where}: 'kv_from' {j} must name an earlier layer")
            src = self.layers[j]
            if src.type != "attention" or src.kv_from is not None:
                raise ConfigError(f"{where}: 'kv_from' {j} must name an attention layer with keys and values of its own")
            if (src.kv_heads, src.dim, src.vdim, src.rot) != (layer.kv_heads, layer.dim, layer.vdim, layer.rot):
                raise ConfigError(f"{where}: layer {j}'s kv_heads, dim, vdim and rot must equal this layer's")

    def to_dict(self) -> dict:
        out = {"architecture": "Fetorax", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "layers": [layer.to_dict() for layer in self.layers]}
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        if self.max_positions != 32768:
            out["max_positions"] = self.max_positions
        return out

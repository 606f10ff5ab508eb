"""The Fetorax decoder, described from parts.

A list of layers, each with its own mixer and sizes: attention (grouped heads, biases
on q, k and v, rotation of a head's first dimensions with linearly scaled frequencies, a
sink in the softmax denominator, a sigmoid output gate, optionally the keys and values
of an earlier layer), retention (a decayed matrix state per head) or mlstm (a gated
matrix state per head).  Every branch is normed before and after
(`parts/block.py: sandwich_norm`) whose tensors hold gain minus one (`rms_norm` with
offset 1); the feed-forward is W_down relu(W_up h)^2 or absent; the logits pass a soft cap.

Tensor names: `embed`, `l<i>.norm1 | norm1b | norm2 | norm2b`, `l<i>.mix.<q|k|v|g|o>`,
biases as `<name>.b`, `l<i>.mix.sink`, `l<i>.mix.norm`, `l<i>.mix.<i|f>`, `l<i>.mlp.<up|down>`,
`final.norm`, `head`.
"""
from __future__ import annotations

from ..config.fetorax import FetoraxConfig, FetoraxLayer
from ..config.registry import register_architecture
from ..parts.rope import LinearScaling
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _norm(cfg: FetoraxConfig, name: str) -> PartSpec:
    return PartSpec("rms_norm", {"size": cfg.width, "eps": cfg.norm_eps, "name": name, "offset": 1.0})


def _position(layer: FetoraxLayer) -> PartSpec | None:
    rot = layer.rot
    if rot is None:
        return None
    return PartSpec("rope", {"head_dim": layer.dim, "theta": rot.base, "rotary_dims": rot.dims,
                             "scaling": LinearScaling(rot.factor) if rot.factor is not None else None})


def _mixer(cfg: FetoraxConfig, layer: FetoraxLayer) -> PartSpec:
    common = {"hidden_size": cfg.width, "n_heads": layer.heads}
    if layer.type == "attention":
        return PartSpec("attention", {
            **common, "n_kv_heads": layer.kv_heads, "head_dim": layer.dim, "value_dim": layer.vdim,
            "scale": layer.scale, "position": _position(layer), "own_kv": layer.kv_from is None,
            "bias": True, "sink": True, "gate": "sigmoid",
            "names": {"q": "mix.q", "k": "mix.k", "v": "mix.v", "o": "mix.o", "g": "mix.g", "sink": "mix.sink",
                      "q_bias": "mix.q.b", "k_bias": "mix.k.b", "v_bias": "mix.v.b"}})
    names = {k: "mix." + k for k in ("q", "k", "v", "g", "o")}
    if layer.type == "retention":
        return PartSpec("retention", {**common, "key_dim": layer.dim, "value_dim": layer.vdim, "decay": layer.decay,
                                      "eps": cfg.norm_eps, "position": _position(layer), "names": names})
    return PartSpec("mlstm", {**common, "key_dim": layer.dim, "value_dim": layer.vdim, "gate_cap": layer.gate_cap,
                              "eps": cfg.norm_eps,
                              "names": {**names, "norm": "mix.norm", "i": "mix.i", "i_bias": "mix.i.b", "f": "mix.f",
                                        "f_bias": "mix.f.b"}})


def describe(cfg: FetoraxConfig) -> ModelSpec:
    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        parts = dict(norm1=_norm(cfg, "norm1"), mixer=_mixer(cfg, layer), norm1b=_norm(cfg, "norm1b"))
        if layer.mlp is not None:
            parts.update(norm2=_norm(cfg, "norm2"), norm2b=_norm(cfg, "norm2b"),
                         ffn=PartSpec("dense_mlp", {"hidden_size": cfg.width, "intermediate_size": layer.mlp.ff,
                                                    "activation": "relu2", "names": {"up": "mlp.up", "down": "mlp.down"}}))
        layers.append(LayerSpec(prefix=f"l{i}.", arrangement="sandwich_norm", parts=parts))
        # A layer without keys and values of its own reads the cache entry of the layer it names.
        if layer.kv_from is not None:
            schedule.append(ScheduleEntry(layer=i, cache=layer.kv_from, writes_cache=False))
        else:
            schedule.append(ScheduleEntry(layer=i, cache=i))
    return ModelSpec(
        name="Fetorax", hidden_size=cfg.width, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "name": "embed"}),
        layers=tuple(layers), schedule=tuple(schedule), final_norm=_norm(cfg, "final.norm"),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "name": "head",
                                      "softcap": cfg.logit_softcap}),
        max_positions=cfg.max_positions)


register_architecture("Fetorax", FetoraxConfig.from_dict, describe)

"""The Zoporax decoder, described from parts.

A list of pre-norm layers, each with its own mixer and sizes: latent attention (queries
through a normed bottleneck; keys and values as per-head maps of one normed latent row per
token plus one rotated key part shared by all heads; YaRN-blended rotation; a sliding window;
a sigmoid output gate) or lightning (a decayed matrix state per head, q, k and v through silu,
one norm over all heads, a sigmoid gate).  The feed-forward is a gated one with biases and the
tanh form of gelu, or routed experts (erf gelu, sigmoid router with groups, a shared expert
behind a scalar gate), or absent.  The head reads the embedding table.

Tensor names: `embed`, `l<i>.norm1 | norm2`, `l<i>.mix.<dq|dq.norm|uq|dkv|dkv.norm|uk|uv|g|o>` or
`l<i>.mix.<q|k|v|g|o|norm>`, `l<i>.mlp.<gate|up|down>` with biases `<name>.b`, or
`l<i>.mlp.router`, `l<i>.mlp.e<j>.<up|down>`, `l<i>.mlp.shared.<up|down|sg>`; `final.norm`.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.zoporax import ZoporaxConfig, ZoporaxLayer
from ..parts.rope import YarnScaling
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _norm(cfg: ZoporaxConfig, name: str) -> PartSpec:
    return PartSpec("rms_norm", {"size": cfg.width, "eps": cfg.norm_eps, "name": name})


def _mixer(cfg: ZoporaxConfig, layer: ZoporaxLayer) -> PartSpec:
    if layer.type == "lightning":
        return PartSpec("lightning", {"hidden_size": cfg.width, "n_heads": layer.heads, "key_dim": layer.dim,
                                      "value_dim": layer.vdim, "decay": layer.decay, "eps": cfg.norm_eps,
                                      "names": {k: "mix." + k for k in ("q", "k", "v", "g", "o", "norm")}})
    position = None
    if layer.rot is not None:
        rot = layer.rot
        scaling = YarnScaling(rot.factor, rot.original, rot.fast, rot.slow) if rot.factor is not None else None
        position = PartSpec("rope", {"head_dim": layer.rot_dim, "theta": rot.base, "rotary_dims": rot.dims, "scaling": scaling})
    return PartSpec("latent_attention", {
        "hidden_size": cfg.width, "n_heads": layer.heads, "head_dim": layer.dim, "rot_dim": layer.rot_dim,
        "value_dim": layer.vdim, "q_rank": layer.q_rank, "kv_rank": layer.kv_rank, "scale": layer.scale,
        "eps": cfg.norm_eps, "position": position, "window": layer.window, "gate": "sigmoid",
        "names": {"dq": "mix.dq", "dq_norm": "mix.dq.norm", "uq": "mix.uq", "dkv": "mix.dkv", "dkv_norm": "mix.dkv.norm",
                  "uk": "mix.uk", "uv": "mix.uv", "g": "mix.g", "o": "mix.o"}})


def _ffn(cfg: ZoporaxConfig, layer: ZoporaxLayer) -> PartSpec:
    mlp = layer.mlp
    if mlp.kind == "dense":
        return PartSpec("gated_mlp", {"hidden_size": cfg.width, "intermediate_size": mlp.ff, "activation": "gelu_tanh", "bias": True,
                                      "names": {"gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down", "gate_bias": "mlp.gate.b",
                                                "up_bias": "mlp.up.b", "down_bias": "mlp.down.b"}})
    r = mlp.router
    return PartSpec("routed_experts", {
        "hidden_size": cfg.width, "n_experts": r.experts, "top": r.top, "expert_size": mlp.ff, "activation": "gelu",
        "groups": r.groups, "keep_groups": r.keep, "route_scale": r.scale, "shared_size": mlp.shared_ff,
        "names": {"router": "mlp.router", "expert": "mlp.e{}", "up": "up", "down": "down", "shared": "mlp.shared",
                  "shared_gate": "mlp.shared.sg"}})


def describe(cfg: ZoporaxConfig) -> ModelSpec:
    layers = []
    for i, layer in enumerate(cfg.layers):
        parts = dict(norm1=_norm(cfg, "norm1"), mixer=_mixer(cfg, layer))
        if layer.mlp is not None:
            parts.update(norm2=_norm(cfg, "norm2"), ffn=_ffn(cfg, layer))
        layers.append(LayerSpec(prefix=f"l{i}.", arrangement="pre_norm", parts=parts))
    return ModelSpec(
        name="Zoporax", hidden_size=cfg.width, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "name": "embed"}),
        layers=tuple(layers), schedule=tuple(ScheduleEntry(layer=i, cache=i) for i in range(len(layers))),
        final_norm=_norm(cfg, "final.norm"),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "name": "head", "tied_to": "embed",
                                      "tied": True}),
        max_positions=cfg.max_positions)


register_architecture("Zoporax", ZoporaxConfig.from_dict, describe)

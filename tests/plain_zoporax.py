"""Plain, slow Zoporax decoder: the oracle that the engine tests of this design compare with.

Whole sequences, no cache, no batching, one function for each mechanism, float64 by
default, token-by-token loops for everything recurrent and for every attention row.
It shares no code with the product: config.json is read as a plain dict, safetensors
with its own few lines, and every formula is written out here.

The design, in this file's notation (h: a mixer's input row, x: the residual stream,
t: a position counted from 0):

  norm(x; w)        x / sqrt(mean(x^2) + eps) * w
  layer             x += mixer(norm1(x));  x += ffn(norm2(x))          (ffn may be absent)
  latent attention  queries through a normed low-rank bottleneck; keys and values expanded, head by
                    head, from one normed latent row per token, plus one rotated key part that all
                    heads share; rotation with YaRN-blended frequencies on the last part of each
                    query head; a sliding causal window; softmax; sigmoid output gate; W_o
  lightning         q, k, v through silu; S_t = g_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; one RMS norm over
                    all heads together, sigmoid gate, W_o
  dense ffn         W_down (gelu_tanh(W_gate h + b_g) * (W_up h + b_u)) + b_d
  routed ffn        sigmoid router scores, the best groups of neighbouring experts by the sum of their two
                    best scores, the best experts inside those groups, weights normalised and scaled; experts
                    W_down gelu(W_up h); a shared expert for every token behind a scalar sigmoid gate
  output            final norm, logits against the embedding table
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch

_ST = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "I32": torch.int32, "I64": torch.int64,
       "F64": torch.float64}


def read_safetensors(path) -> dict[str, torch.Tensor]:
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        dt = _ST[info["dtype"]]
        t = torch.frombuffer(bytearray(raw[8 + n + lo:8 + n + hi]), dtype=dt) if hi > lo else torch.empty(0, dtype=dt)
        out[name] = t.reshape(info["shape"]).clone()
    return out


def load_folder(folder):
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), read_safetensors(folder / "model.safetensors")


# --------------------------------------------------------------------------- small pieces

_STORAGE = None        # set by forward(storage=...): the dtype in which activations are kept between operations


def _st(x: torch.Tensor) -> torch.Tensor:
    """x as an engine that stores its activations in `_STORAGE` would hand it on (the yardstick for bfloat16)."""
    return x if _STORAGE is None else x.to(_STORAGE).to(x.dtype)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


# --------------------------------------------------------------------------- rotation

def yarn_frequencies(dims: int, base: float, scaling: dict | None) -> tuple[torch.Tensor, float]:
    """(f_i for i < dims / 2, the factor on cos and sin)."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.tensor(float(base), dtype=torch.float64) ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turn_dim(turns):        # the dimension whose wave makes `turns` turns over the original length
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(turn_dim(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, pos: int, freqs: torch.Tensor, mult: float) -> torch.Tensor:
    """x [..., dims]: dimension i pairs with i + dims / 2."""
    half = freqs.numel()
    a = pos * freqs
    c, s = (torch.cos(a) * mult).to(x.dtype), (torch.sin(a) * mult).to(x.dtype)
    u, v = x[..., :half], x[..., half:2 * half]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., 2 * half:]], dim=-1)


# --------------------------------------------------------------------------- mixers

def latent_attention(h: torch.Tensor, w: dict, m: dict, eps: float) -> torch.Tensor:
    """h [T, D] -> [T, D].  w: the mixer's tensors by their short names."""
    T = h.shape[0]
    H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = m.get("rot") or {}
    freqs, mult = yarn_frequencies(rot.get("dims", dr), rot["base"], rot.get("scaling")) if rot else (None, 1.0)
    window = (m.get("mask") or {}).get("size")
    cq = _st(rms_norm(h @ w["dq"].T, w["dq.norm"], eps))
    q = _st(cq @ w["uq"].T).reshape(T, H, dn + dr)
    down = h @ w["dkv"].T
    c = _st(rms_norm(down[:, :R], w["dkv.norm"], eps))
    k_shared = down[:, R:]
    k_plain = _st(c @ w["uk"].T).reshape(T, H, dn)
    val = _st(c @ w["uv"].T).reshape(T, H, dv)
    gate = torch.sigmoid(_st(h @ w["g"].T))
    q_rot = torch.stack([rotate(q[t, :, dn:], t, freqs, mult) for t in range(T)]) if rot else q[:, :, dn:]
    k_rot = _st(torch.stack([rotate(k_shared[t], t, freqs, mult) for t in range(T)]) if rot else k_shared)
    q_rot = _st(q_rot)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        first = 0 if window is None else max(0, t - window + 1)
        for a in range(H):
            s = (k_plain[first:t + 1, a] @ q[t, a, :dn] + k_rot[first:t + 1] @ q_rot[t, a]) * m["scale"]
            p = torch.softmax(s, dim=0)
            out[t, a] = p @ val[first:t + 1, a]
    return _st(_st(out.reshape(T, H * dv)) * gate) @ w["o"].T


def lightning(h: torch.Tensor, w: dict, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(_st(h @ w["q"].T)).reshape(T, H, dk)
    k = silu(_st(h @ w["k"].T)).reshape(T, H, dk)
    v = silu(_st(h @ w["v"].T)).reshape(T, H, dv)
    decay = torch.tensor(m["decay"], dtype=h.dtype)
    state = torch.zeros(H, dk, dv, dtype=h.dtype)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        state = decay[:, None, None] * state + k[t, :, :, None] * v[t, :, None, :]
        out[t] = torch.einsum("hkv,hk->hv", state, q[t])
    y = rms_norm(out.reshape(T, H * dv), w["norm"], eps) * torch.sigmoid(_st(h @ w["g"].T))
    return _st(y) @ w["o"].T


# --------------------------------------------------------------------------- feed-forwards

def dense_ffn(h: torch.Tensor, w: dict) -> torch.Tensor:
    a = gelu_tanh(h @ w["gate"].T + w["gate.b"]) * (h @ w["up"].T + w["up.b"])
    return _st(a) @ w["down"].T + w["down.b"]


def expert(h: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return _st(gelu_erf(_st(h @ up.T))) @ down.T


_MARGINS = None        # set by forward(margins_out=...): receives, per routed layer, every token's narrowest choice


def choice_margin(scores: torch.Tensor, router: dict) -> float:
    """How far the token's choice is from another one: the smallest gap, in score, between what was just taken and
    what was just left (the last kept and the first dropped group, by the groups' scores; the last chosen and the
    first unchosen expert of the kept groups).  Infinite when nothing is left out."""
    E, top = router["experts"], router["top"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    per = E // groups["count"]
    margin = float("inf")
    group_score = scores.reshape(groups["count"], per).topk(min(2, per), dim=1).values.sum(dim=1)
    ranked = group_score.sort(descending=True)
    if groups["keep"] < groups["count"]:
        margin = float(ranked.values[groups["keep"] - 1] - ranked.values[groups["keep"]])
    kept = ranked.indices[:groups["keep"]].tolist()
    inside = torch.cat([scores[g * per:(g + 1) * per] for g in kept]).sort(descending=True).values
    if top < inside.numel():
        margin = min(margin, float(inside[top - 1] - inside[top]))
    return margin


def route(scores: torch.Tensor, router: dict) -> tuple[list[int], torch.Tensor]:
    """scores [E] of one token -> (chosen experts, their weights)."""
    E, top = router["experts"], router["top"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    per = E // groups["count"]
    by_group = scores.reshape(groups["count"], per)
    group_score = by_group.topk(min(2, per), dim=1).values.sum(dim=1)
    kept = group_score.topk(groups["keep"]).indices.tolist()
    allowed = torch.full((E,), False)
    for g in kept:
        allowed[g * per:(g + 1) * per] = True
    masked = torch.where(allowed, scores, torch.full_like(scores, -1.0))       # scores are sigmoids: all above zero
    chosen = masked.topk(top).indices.tolist()
    weights = scores[chosen]
    return chosen, weights / (weights.sum() + 1e-20) * router.get("scale", 1.0)


def routed_ffn(h: torch.Tensor, w: dict, mlp: dict) -> torch.Tensor:
    router = mlp["router"]
    T = h.shape[0]
    out = torch.zeros(T, w["e0.down"].shape[0], dtype=h.dtype)
    scores = torch.sigmoid(h @ w["router"].T)
    if _MARGINS is not None:
        _MARGINS.append(torch.tensor([choice_margin(scores[t], router) for t in range(T)], dtype=torch.float64))
    for t in range(T):
        chosen, weights = route(scores[t], router)
        for e, g in zip(chosen, weights):
            out[t] += g * expert(h[t], w[f"e{e}.up"], w[f"e{e}.down"])
    if mlp.get("shared"):
        out += torch.sigmoid(h @ w["shared.sg"].T) * expert(h, w["shared.up"], w["shared.down"])
    return out


# --------------------------------------------------------------------------- the model

def _sub(weights: dict, prefix: str, dtype) -> dict:
    return {k[len(prefix):]: v.to(dtype) for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg: dict, weights: dict, tokens, dtype=torch.float64, storage=None, layers_out: list | None = None,
            margins_out: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence.  storage: keep activations in this dtype between operations (everything
    else stays in `dtype`).  layers_out: receives the residual stream after every layer.  margins_out: receives, for
    every routed layer, each token's `choice_margin`."""
    global _STORAGE, _MARGINS
    _STORAGE, _MARGINS = storage, margins_out
    try:
        eps = cfg["norm"]["eps"]
        embed = weights["embed"].to(dtype)
        x = embed[torch.tensor(list(tokens), dtype=torch.long)]
        for i, layer in enumerate(cfg["layers"]):
            p = f"l{i}."
            mix = _sub(weights, p + "mix.", dtype)
            h = _st(rms_norm(x, weights[p + "norm1"].to(dtype), eps))
            if layer["type"] == "latent_attention":
                x = x + latent_attention(h, mix, layer["mixer"], eps)
            elif layer["type"] == "lightning":
                x = x + lightning(h, mix, layer["mixer"], eps)
            else:
                raise ValueError(layer["type"])
            mlp = layer.get("mlp")
            if mlp is not None:
                h = _st(rms_norm(x, weights[p + "norm2"].to(dtype), eps))
                ff = _sub(weights, p + "mlp.", dtype)
                x = x + (dense_ffn(h, ff) if mlp["kind"] == "dense" else routed_ffn(h, ff, mlp))
            if layers_out is not None:
                layers_out.append(x.clone())
        return _st(rms_norm(x, weights["final.norm"].to(dtype), eps)) @ embed.T
    finally:
        _STORAGE = _MARGINS = None


def greedy(cfg: dict, weights: dict, prompt, n_new: int) -> list[int]:
    seq = list(prompt)
    for _ in range(n_new):
        seq.append(int(forward(cfg, weights, seq)[-1].argmax()))
    return seq[len(prompt):]

"""Plain, slow Fetorax decoder: the oracle that the engine tests of this design compare with.

Whole sequences, no cache, no batching, one function for each mechanism, float64
by default, token-by-token loops for everything recurrent.  It shares no code with
the product: config.json is read as a plain dict, safetensors with its own few
lines, and every formula is written out here.

The design, in this file's notation (h: a mixer's input row, x: the residual stream,
t: a position counted from 0, D_h: a head's key size):

  norm(x; w)      x / sqrt(mean(x^2) + eps) * (1 + w)
  layer           x += norm1b(mixer(norm1(x)));  x += norm2b(ffn(norm2(x)))   (ffn may be absent)
  ffn             W_down relu(W_up h)^2
  attention       q, k, v with biases; partial rotary with linearly scaled frequencies;
                  p_j = exp(s_j) / (exp(sink) + sum_j' exp(s_j')); sigmoid output gate; W_o;
                  optionally reading another layer's keys and values
  retention       S_t = g S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, unit RMS per head, silu gate, W_o
  mlstm           stabilised matrix memory with exponential input gate and sigmoid forget gate
  output          final norm, head, soft cap c tanh(z / c)
"""
from __future__ import annotations

import json
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


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The tensor holds the gain minus one."""
    return unit_rms(x, eps) * (1.0 + w)


def relu_squared_ffn(h: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    a = torch.clamp(_st(h @ up.T), min=0.0)
    return _st(a * a) @ down.T


def rotary_frequencies(dims: int, base: float, factor: float | None) -> torch.Tensor:
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.tensor(float(base), dtype=torch.float64) ** (-2.0 * i / dims)
    return f / factor if factor else f


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: dict | None) -> torch.Tensor:
    """x [T, heads, size]: the first rot.dims of each head in pairs (i, i + dims/2); the rest pass."""
    if not rot or not rot.get("dims"):
        return x
    dims = int(rot["dims"])
    factor = (rot.get("scaling") or {}).get("factor")
    ang = positions.to(torch.float64)[:, None] * rotary_frequencies(dims, rot["base"], factor)[None, :]
    c, s = torch.cos(ang)[:, None, :].to(x.dtype), torch.sin(ang)[:, None, :].to(x.dtype)
    u, v = x[..., :dims // 2], x[..., dims // 2:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def softcap(z: torch.Tensor, cap: float | None) -> torch.Tensor:
    return cap * torch.tanh(z / cap) if cap else z


# --------------------------------------------------------------------------- mixers

def attention_keys_values(h, m: dict, w: dict, pre: str):
    """The rotated keys and the values of a layer that has projections of its own: [T, G, size]."""
    T = h.shape[0]
    G, dk, dv = m["kv_heads"], m["dim"], m["vdim"]
    k = (h @ w[pre + "k"].T + w[pre + "k.b"]).reshape(T, G, dk)
    v = (h @ w[pre + "v"].T + w[pre + "v.b"]).reshape(T, G, dv)
    return _st(rotate(k, torch.arange(T), m.get("rot"))), _st(v)


def sink_attention(h, m: dict, w: dict, pre: str, k, v) -> torch.Tensor:
    """Causal grouped attention over given keys and values, with one more term exp(sink) in every
    head's denominator, gated by sigmoid(W_g h) before the output projection."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = _st(rotate((h @ w[pre + "q"].T + w[pre + "q.b"]).reshape(T, H, dk), torch.arange(T), m.get("rot")))
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        for t in range(T):
            s = (k[:t + 1, g] @ q[t, head]) * m["scale"]
            sink = w[pre + "sink"][head]
            top = torch.maximum(s.max(), sink)
            e = torch.exp(s - top)
            out[t, head] = (e[:, None] * v[:t + 1, g]).sum(0) / (e.sum() + torch.exp(sink - top))
    gate = torch.sigmoid(_st(h @ w[pre + "g"].T))
    return _st(out.reshape(T, H * dv) * gate) @ w[pre + "o"].T


def retention(h, m: dict, w: dict, pre: str, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = rotate(_st(h @ w[pre + "q"].T).reshape(T, H, dk), pos, m.get("rot"))
    k = rotate(_st(h @ w[pre + "k"].T).reshape(T, H, dk), pos, m.get("rot")) * dk ** -0.5
    v = _st(h @ w[pre + "v"].T).reshape(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for head in range(H):
        S = torch.zeros(dk, dv, dtype=h.dtype)
        for t in range(T):
            S = m["decay"][head] * S + torch.outer(k[t, head], v[t, head])
            out[t, head] = S.T @ q[t, head]
    out = unit_rms(out, eps).reshape(T, H * dv)
    return _st(out * torch.nn.functional.silu(_st(h @ w[pre + "g"].T))) @ w[pre + "o"].T


def mlstm(h, m: dict, w: dict, pre: str, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, dk, dv, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = _st(h @ w[pre + "q"].T).reshape(T, H, dk) * dk ** -0.5
    k = _st(h @ w[pre + "k"].T).reshape(T, H, dk)
    v = _st(h @ w[pre + "v"].T).reshape(T, H, dv)
    log_i = cap * torch.tanh((h @ w[pre + "i"].T + w[pre + "i.b"]) / cap)                                     # [T, H]
    log_f = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w[pre + "f"].T + w[pre + "f.b"]) / cap))
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for head in range(H):
        S, n, mx = torch.zeros(dk, dv, dtype=h.dtype), torch.zeros(dk, dtype=h.dtype), torch.zeros((), dtype=h.dtype)
        for t in range(T):
            new_mx = torch.maximum(log_f[t, head] + mx, log_i[t, head])
            keep, take = torch.exp(log_f[t, head] + mx - new_mx), torch.exp(log_i[t, head] - new_mx)
            S = keep * S + take * torch.outer(k[t, head], v[t, head])
            n = keep * n + take * k[t, head]
            mx = new_mx
            out[t, head] = S.T @ q[t, head] / (torch.maximum(torch.abs(n @ q[t, head]), torch.exp(-mx)) + 1e-6)
    out = unit_rms(out, eps).reshape(T, H * dv) * w[pre + "norm"]
    return _st(out * torch.sigmoid(_st(h @ w[pre + "g"].T))) @ w[pre + "o"].T


# --------------------------------------------------------------------------- the model

def forward(cfg: dict, weights: dict, tokens, dtype=torch.float64, layers_out: list | None = None,
            storage=None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence; `layers_out` collects the residual stream after every layer.
    storage=torch.bfloat16 rounds what an engine of that precision keeps between its operations (the rows a
    norm hands on, projections, a mixer's output before its last product, the feed-forward's hidden rows);
    the residual stream, the norms, scores and states stay exact."""
    global _STORAGE
    _STORAGE = storage
    try:
        return _forward(cfg, weights, tokens, dtype, layers_out)
    finally:
        _STORAGE = None


def _forward(cfg, weights, tokens, dtype, layers_out):
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    kept: dict[int, tuple] = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = _st(offset_norm(x, w[p + "norm1"], eps))
        kind = layer["type"]
        if kind == "attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = attention_keys_values(h, m, w, p + "mix.")
                src = i
            y = sink_attention(h, m, w, p + "mix.", *kept[src])
        elif kind == "retention":
            y = retention(h, m, w, p + "mix.", eps)
        elif kind == "mlstm":
            y = mlstm(h, m, w, p + "mix.", eps)
        else:
            raise ValueError(f"layer {i}: unknown mixer {kind!r}")
        x = x + offset_norm(y, w[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            h = _st(offset_norm(x, w[p + "norm2"], eps))
            x = x + offset_norm(relu_squared_ffn(h, w[p + "mlp.up"], w[p + "mlp.down"]), w[p + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    z = _st(offset_norm(x, w["final.norm"], eps)) @ w["head"].T
    return softcap(z, cfg.get("logit_softcap"))


def greedy(cfg: dict, weights: dict, prompt, n_new: int, stop=()) -> list[int]:
    """Greedy continuation by running the whole sequence again for every token."""
    seq, out = list(prompt), []
    for _ in range(n_new):
        tok = int(forward(cfg, weights, seq)[-1].argmax())
        if tok in stop:
            break
        out.append(tok)
        seq.append(tok)
    return out

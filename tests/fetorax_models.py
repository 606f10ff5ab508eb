"""Small Fetorax configurations and model folders with random weights, for the tests of this design.

The configurations differ from each other in every size and option: groups of 3, 1 and 2 heads per
kv head; values wider and narrower than keys; rotation of a few, of half and of all of a head's
dimensions, with and without frequency scaling; layers without a feed-forward; two layers that read
an earlier layer's keys and values; key sizes of the recurrent mixers that take each variant of the
scan kernel (up to 64, 128, 256); a width that is no multiple of 8; with and without a logit cap.
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

import plain_fetorax


def attention(heads, kv_heads, dim, vdim, rot=None, scale=None, kv_from=None, ff=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5 if scale is None else scale}
    if rot is not None:
        m["rot"] = rot
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def retention(heads, dim, vdim, decay, rot=None, ff=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}
    if rot is not None:
        m["rot"] = rot
    return {"type": "retention", "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def mlstm(heads, dim, vdim, gate_cap, ff=None):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": gate_cap},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def model(width, vocab, layers, eps=1e-5, softcap=None):
    out = {"architecture": "Fetorax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if softcap is not None:
        out["logit_softcap"] = softcap
    return out


ROT_A = {"dims": 8, "base": 10000.0, "scaling": {"factor": 4.0}}
ROT_FULL = {"dims": 32, "base": 500.0}

CONFIGS = {
    # every mixer, groups of three, narrow values, a layer without feed-forward, shared keys and values
    "mixed": model(64, 200, [
        attention(6, 2, 32, 16, rot=ROT_A, scale=0.2, ff=96),
        retention(2, 16, 24, [0.9, 0.99], rot={"dims": 8, "base": 300.0}),
        mlstm(3, 24, 40, 8.0, ff=80),
        attention(6, 2, 32, 16, rot=ROT_A, scale=0.2, kv_from=0),
        attention(2, 2, 32, 32, rot=ROT_FULL, ff=64),
        attention(2, 2, 32, 32, rot=ROT_FULL, scale=0.3, kv_from=4, ff=72),
    ], eps=1e-6, softcap=20.0),
    # one head everywhere, a width that is no multiple of 8, no rotation in the attention, no logit cap,
    # key sizes 72 and 136 (the wider variants of the scan kernel), values wider than keys
    "odd": model(100, 131, [
        mlstm(1, 72, 20, 15.0),
        attention(1, 1, 24, 40, ff=50),
        retention(1, 136, 12, [0.97], ff=60),
    ], eps=1e-5),
    # the head size of real models (64) with two heads per kv head, decays close to one
    "head64": model(128, 300, [
        attention(4, 2, 64, 64, rot={"dims": 32, "base": 1e6, "scaling": {"factor": 2.0}}, scale=0.125, ff=192),
        retention(2, 64, 64, [0.996, 0.9995], rot={"dims": 64, "base": 1e4}, ff=192),
        mlstm(2, 64, 64, 10.0, ff=192),
        attention(4, 2, 64, 64, rot={"dims": 32, "base": 1e6, "scaling": {"factor": 2.0}}, scale=0.125, kv_from=0, ff=192),
    ], softcap=30.0),
    # head size 128 with three heads on one kv head, and head size 64 with a kv head for every head: the groups
    # of odd size, which the tensor-core prompt kernel serves one head per block
    "odd_groups": model(128, 210, [
        attention(3, 1, 128, 128, rot={"dims": 64, "base": 5e5, "scaling": {"factor": 8.0}}, scale=0.09, ff=160),
        attention(2, 2, 64, 64, rot={"dims": 64, "base": 1e4}, scale=0.11),
        attention(3, 1, 128, 128, rot={"dims": 64, "base": 5e5, "scaling": {"factor": 8.0}}, scale=0.2, kv_from=0, ff=96),
    ], eps=1e-5, softcap=25.0),
    # one layer of each mixer alone, without feed-forward
    "only_attention": model(48, 90, [attention(4, 1, 16, 24, rot={"dims": 16, "base": 100.0, "scaling": {"factor": 1.5}}, scale=0.4)]),
    "only_retention": model(48, 90, [retention(3, 16, 8, [0.8, 0.95, 0.999], rot={"dims": 4, "base": 50.0})]),
    "only_mlstm": model(48, 90, [mlstm(2, 8, 16, 5.0)], softcap=12.0),
}


def make_folder(tmp, name: str, seed: int = 0, std: float = 0.1, gain_std: float = 0.2, dtype=torch.bfloat16) -> Path:
    """A model folder with random weights, written by the framework's random-weights mode."""
    import longbow_quarrel_b200  # noqa: F401
    from longbow_quarrel_b200 import architectures  # noqa: F401
    from longbow_quarrel_b200.config import architecture_of
    from longbow_quarrel_b200.engine.model import Model
    from longbow_quarrel_b200.parts.base import Runtime
    from longbow_quarrel_b200.weights import write_random_model
    data = CONFIGS[name] if isinstance(name, str) else name
    arch = architecture_of(data)
    cfg = arch.config_from_dict(data)
    table = Model(arch.describe(cfg), Runtime(torch.device("cpu"), torch.float32, 64)).weight_table()
    label = name if isinstance(name, str) else "custom"
    return write_random_model(Path(tmp) / f"fetorax_{label}_{seed}", cfg.to_dict(), table, seed, dtype, std, gain_std)


def tokens(n: int, vocab: int, seed: int) -> list[int]:
    return [int(t) for t in np.random.default_rng(seed).integers(0, vocab, size=n)]


def row_errors(got: np.ndarray, ref: np.ndarray) -> np.ndarray:
    """Per row: root mean square of the difference over the root mean square of the reference row."""
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert np.isfinite(got).all(), "non-finite logits"
    return np.sqrt(((got - ref) ** 2).mean(-1)) / np.maximum(np.sqrt((ref ** 2).mean(-1)), 1e-30)


F32_TOL = 2e-5        # the floor of every float32 bound, per row


def bound(dtype: str, cfg: dict, weights: dict, toks, exact: np.ndarray) -> float:
    """What a row may differ by from the float64 plain implementation, measured on the request itself and not
    assumed.  float32: three times what the plain implementation moves by when it runs in float32 (a unit norm
    of a nearly cancelled sum makes single positions of some requests ten times worse than others), at least
    2e-5.  bfloat16: three times what it moves by when it keeps its activations in bfloat16.  Both take the
    request's worst row."""
    if dtype == "float32":
        single = plain_fetorax.forward(cfg, weights, toks, dtype=torch.float32).numpy()
        return max(F32_TOL, 3.0 * float(row_errors(single, exact).max()))
    stored = plain_fetorax.forward(cfg, weights, toks, storage=torch.bfloat16).numpy()
    return 3.0 * float(row_errors(stored, exact).max())


def load(folder):
    return json.loads((Path(folder) / "config.json").read_text()), plain_fetorax.read_safetensors(Path(folder) / "model.safetensors")

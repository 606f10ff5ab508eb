"""Small Zoporax configurations and model folders with random weights, for the tests of this design.

The configurations differ from each other in every size and option: windows of 5, 33, 64 and 100 tokens and
no window; rotation of all and of a part of the rotated size, with and without YaRN blending (ramps that
cover all, some and none of the dimensions); latents that are no multiple of 32; one head; values wider and
narrower than keys; experts in 1, 2 and 4 groups of which 1, 2 or all are kept, 1 to 3 experts per token, with
and without a shared expert; layers without a feed-forward; a width that is no multiple of 8.
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

import plain_zoporax


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, window=None, rot=None, scale=None, mlp=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "scale": (dim + rot_dim) ** -0.5 if scale is None else scale}
    if window is not None:
        m["mask"] = {"size": window}
    if rot is not None:
        m["rot"] = rot
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def lightning(heads, dim, vdim, decay, mlp=None):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, groups=None, scale=1.0, shared=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def model(width, vocab, layers, eps=1e-5):
    return {"architecture": "Zoporax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


YARN_A = {"dims": 8, "base": 10000.0, "scaling": {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}}
YARN_B = {"dims": 24, "base": 1e6, "scaling": {"factor": 8.0, "original": 256, "fast": 32.0, "slow": 1.0}}
ROT_PLAIN = {"dims": 16, "base": 500.0}

CONFIGS = {
    # both mixers and all three feed-forwards; a window of 33 (just over half a page) and one of 100 (more than a page)
    "mixed": model(64, 200, [
        latent(3, 16, 8, 24, 40, 24, window=33, rot=YARN_A, scale=0.3, mlp=moe(6, 2, 32, groups=(3, 2), scale=1.7, shared=48)),
        lightning(2, 16, 24, [0.9, 0.995], mlp=dense(96)),
        latent(2, 24, 16, 8, 32, 40, window=100, rot=ROT_PLAIN, mlp=None),
        lightning(3, 8, 8, [0.5, 0.97, 1.0], mlp=moe(4, 1, 40, scale=2.0)),
        latent(3, 16, 8, 24, 40, 24, window=33, rot=YARN_A, scale=0.3, mlp=dense(72)),
    ], eps=1e-6),
    # one head everywhere, a width that is no multiple of 8, a latent of 20, no window, a rotation that leaves a part of
    # the rotated size alone, a router without groups whose every expert is used
    "odd": model(100, 131, [
        latent(1, 12, 12, 20, 28, 20, rot={"dims": 8, "base": 300.0}, mlp=moe(3, 3, 24, shared=16)),
        lightning(1, 40, 12, [0.98]),
        latent(1, 12, 12, 20, 28, 20, window=5, rot={"dims": 8, "base": 300.0}, mlp=dense(50)),
    ]),
    # sizes near those of real layers, small: eight heads, a latent of 96, a window of exactly one page
    "wide": model(128, 300, [
        lightning(4, 32, 64, [0.8, 0.95, 0.99, 0.999], mlp=moe(16, 3, 48, groups=(4, 2), scale=2.5, shared=64)),
        latent(8, 32, 24, 16, 96, 96, window=64, rot=YARN_B, scale=0.12, mlp=moe(16, 3, 48, groups=(4, 2), scale=2.5, shared=64)),
        latent(8, 32, 24, 16, 96, 96, window=64, rot=YARN_B, scale=0.12, mlp=dense(192)),
    ]),
    # one layer of each mixer alone, without feed-forward; and each feed-forward behind the cheapest mixer
    "only_latent": model(48, 90, [latent(4, 8, 8, 12, 24, 16, window=20, rot={"dims": 8, "base": 100.0, "scaling": {
        "factor": 2.0, "original": 32, "fast": 8.0, "slow": 1.0}}, scale=0.4)]),
    "only_latent_full": model(48, 90, [latent(2, 16, 4, 8, 16, 36, rot={"dims": 4, "base": 50.0})]),
    # sizes that no tensor-core kernel takes (cache rows of 26 numbers, heads of 10 + 6): the plain kernels in bfloat16 too
    "only_latent_ragged": model(44, 90, [latent(3, 10, 6, 14, 20, 20, window=17, rot={"dims": 4, "base": 200.0, "scaling": {
        "factor": 3.0, "original": 16, "fast": 4.0, "slow": 1.0}}, scale=0.3, mlp=moe(4, 2, 12, groups=(2, 1), shared=20))]),
    "only_lightning": model(48, 90, [lightning(3, 16, 8, [0.7, 0.95, 0.999])]),
    "only_dense": model(40, 70, [lightning(1, 8, 8, [0.9], mlp=dense(56))]),
    "only_moe": model(40, 70, [lightning(1, 8, 8, [0.9], mlp=moe(8, 2, 16, groups=(4, 1), scale=0.5, shared=24))]),
    "only_moe_plain": model(40, 70, [lightning(1, 8, 8, [0.9], mlp=moe(5, 2, 16))]),
}


def make_folder(tmp, name, seed: int = 0, std: float = 0.1, gain_std: float = 0.2, dtype=torch.bfloat16) -> Path:
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
    return write_random_model(Path(tmp) / f"zoporax_{label}_{seed}", cfg.to_dict(), table, seed, dtype, std, gain_std)


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
    """What a row may differ by from the float64 plain implementation, measured on the request itself: three times
    what the plain implementation moves by when it runs in float32 (at least 2e-5), or when it keeps its
    activations in bfloat16.  Both take the request's worst row."""
    if dtype == "float32":
        single = plain_zoporax.forward(cfg, weights, toks, dtype=torch.float32).numpy()
        return max(F32_TOL, 3.0 * float(row_errors(single, exact).max()))
    stored = plain_zoporax.forward(cfg, weights, toks, storage=torch.bfloat16).numpy()
    return 3.0 * float(row_errors(stored, exact).max())


def load(folder):
    return json.loads((Path(folder) / "config.json").read_text()), plain_zoporax.read_safetensors(Path(folder) / "model.safetensors")


CLOSE_CALL = 0.02      # in score (a sigmoid): rounding in bfloat16 moves a router's scores by a few thousandths


def firm_rows(dtype: str, cfg: dict, weights: dict, toks) -> np.ndarray:
    """Which positions' logits a bfloat16 run can be held to: those where no router's choice is a close call.  Where two
    experts (or two groups) score within CLOSE_CALL of each other at the edge of the choice, rounding decides which
    one is taken, and the row that follows is another row; both are right.  float32: every position."""
    firm = np.ones(len(toks), dtype=bool)
    if dtype != "float32":
        margins: list = []
        plain_zoporax.forward(cfg, weights, toks, margins_out=margins)
        for m in margins:
            firm &= m.numpy() >= CLOSE_CALL
    return firm

"""Zoporax without a GPU: the typed configuration and its errors, the model as data (which storage each mixer
asks for), the weight table, the rotation tables, and the plain implementation against itself."""
import copy
import math

import pytest
import torch

import plain_zoporax
from zoporax_models import CONFIGS, load, make_folder, row_errors, tokens


def _arch(data):
    import longbow_quarrel_b200  # noqa: F401
    from longbow_quarrel_b200 import architectures  # noqa: F401
    from longbow_quarrel_b200.config import architecture_of
    arch = architecture_of(data)
    return arch, arch.config_from_dict(data)


def test_configuration_round_trip_and_description():
    from longbow_quarrel_b200.parts.base import KVNeed, Runtime, StateNeed
    from longbow_quarrel_b200.engine.model import Model
    arch, cfg = _arch(CONFIGS["mixed"])
    assert arch.name == "Zoporax"
    assert _arch(cfg.to_dict())[1] == cfg
    assert cfg.layers[0].rot.factor == 4.0 and cfg.layers[2].rot.factor is None and cfg.layers[2].mlp is None
    assert cfg.layers[0].mlp.router.groups == 3 and cfg.layers[3].mlp.router.groups == 1 and cfg.layers[3].mlp.shared_ff is None
    spec = arch.describe(cfg)
    assert [(e.layer, e.cache, e.writes_cache) for e in spec.schedule] == [(i, i, True) for i in range(5)]
    model = Model(spec, Runtime(torch.device("cpu"), torch.float32, 128))
    needs = model.cache_needs()
    # One row of latent + shared key part per token, no pool of values; the windows group the entries.
    assert needs[0] == KVNeed(1, 24 + 8, 33, None, False) == needs[4] and needs[2] == KVNeed(1, 40 + 16, 100, None, False)
    assert needs[1] == StateNeed((2, 16, 24)) and needs[3] == StateNeed((3, 8, 8))
    table = model.weight_table()
    assert table["l0.mix.dq"].shape == (40, 64) and table["l0.mix.uq"].shape == (3 * 24, 40) and table["l0.mix.dkv"].shape == (32, 64)
    assert table["l0.mix.uk"].shape == (48, 24) and table["l0.mix.uv"].shape == (72, 24) and table["l0.mix.o"].shape == (64, 72)
    assert table["l0.mix.dq.norm"].shape == (40,) and table["l0.mix.dkv.norm"].shape == (24,) and table["l0.mix.g"].shape == (72, 64)
    assert table["l1.mix.norm"].shape == (48,) and table["l1.mlp.gate.b"].shape == (96,) and table["l1.mlp.down.b"].shape == (64,)
    assert table["l0.mlp.router"].shape == (6, 64) and table["l0.mlp.e5.up"].shape == (32, 64) and "l0.mlp.e6.up" not in table
    assert table["l0.mlp.shared.up"].shape == (48, 64) and table["l0.mlp.shared.sg"].shape == (1, 64)
    assert "l3.mlp.shared.up" not in table and "l2.norm2" not in table and "l2.mlp.up" not in table
    assert "head" not in table and "final.norm" in table
    assert model.graph_safe and model.kernel_libraries() == ("latent_attn", "moe", "recurrent")


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), "at most"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("fast"), "fast"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "size"),
    (lambda c: c["layers"][2].update(type="attention"), "not one of"),
    (lambda c: c["layers"][1]["mlp"].update(kind="routed"), "not supported"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(experts=7), "equal groups"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "top"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(keep=4), "kept"),
    (lambda c: c["layers"][0]["mlp"].pop("expert"), "expert"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.update(layers=[]), "layers"),
])
def test_configuration_errors_name_the_key(change, word):
    from longbow_quarrel_b200.config import ConfigError
    data = copy.deepcopy(CONFIGS["mixed"])
    change(data)
    with pytest.raises(ConfigError, match=word):
        _arch(data)


@pytest.mark.parametrize("dims,base,scaling", [
    (8, 10000.0, {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}),      # the ramp covers some dimensions
    (24, 1e6, {"factor": 8.0, "original": 256, "fast": 32.0, "slow": 1.0}),
    (16, 100.0, {"factor": 2.0, "original": 4096, "fast": 4.0, "slow": 1.0}),        # every dimension is fast: lo = hi
    (6, 5e5, {"factor": 3.0, "original": 8, "fast": 64.0, "slow": 32.0}),            # every dimension is slow
    (12, 300.0, None),
])
def test_rotation_tables_follow_the_blend(dims, base, scaling):
    """The framework's tables against the frequencies written out here: blended between f and f / factor along a
    ramp over the dimension index, cos and sin both times 0.1 ln(factor) + 1."""
    from longbow_quarrel_b200.parts.base import Runtime
    from longbow_quarrel_b200.parts.registry import make_part
    from longbow_quarrel_b200.parts.rope import YarnScaling
    from longbow_quarrel_b200.parts.spec import PartSpec
    sc = YarnScaling(scaling["factor"], scaling["original"], scaling["fast"], scaling["slow"]) if scaling else None
    part = make_part("position", PartSpec("rope", {"head_dim": dims + 4, "theta": base, "rotary_dims": dims, "scaling": sc}),
                     Runtime(torch.device("cpu"), torch.float32, 200))
    cos, sin = part.tables()
    freqs, mult = plain_zoporax.yarn_frequencies(dims, base, scaling)
    pos = torch.arange(200, dtype=torch.float64)[:, None]
    assert cos.shape == (200, dims // 2)
    assert (cos.double() - torch.cos(pos * freqs) * mult).abs().max() < 1e-6
    assert (sin.double() - torch.sin(pos * freqs) * mult).abs().max() < 1e-6
    if scaling:
        plain = torch.tensor(base, dtype=torch.float64) ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims)
        assert (freqs <= plain * (1 + 1e-12)).all() and (freqs >= plain / scaling["factor"] * (1 - 1e-12)).all()
        assert mult == pytest.approx(0.1 * math.log(scaling["factor"]) + 1.0)


def test_routing_of_the_plain_implementation():
    """Scores chosen so that the group rule shows: the best single expert sits in a group whose two best
    together lose, so it must not be chosen."""
    router = {"experts": 6, "top": 2, "scale": 2.0, "groups": {"count": 3, "keep": 1}}
    scores = torch.tensor([0.95, 0.05, 0.6, 0.55, 0.1, 0.2], dtype=torch.float64)
    chosen, weights = plain_zoporax.route(scores, router)
    assert sorted(chosen) == [2, 3]
    assert float(weights.sum()) == pytest.approx(2.0) and float(weights[chosen.index(2)]) == pytest.approx(2.0 * 0.6 / 1.15)
    chosen, _ = plain_zoporax.route(scores, {**router, "groups": {"count": 3, "keep": 2}})
    assert sorted(chosen) == [0, 2]
    chosen, _ = plain_zoporax.route(scores, {"experts": 6, "top": 3, "scale": 1.0})
    assert sorted(chosen) == [0, 2, 3]


def test_plain_implementation_agrees_with_itself(tmp_path):
    """A prefix's logits do not depend on what follows; float32 stays close to float64; a token beyond a window
    no longer changes a later position in a model of latent attention alone, while one inside it does."""
    folder = make_folder(tmp_path, "mixed", seed=1)
    cfg, weights = load(folder)
    toks = tokens(60, cfg["vocab"], 2)
    full = plain_zoporax.forward(cfg, weights, toks).numpy()
    part = plain_zoporax.forward(cfg, weights, toks[:17]).numpy()
    assert row_errors(part, full[:17]).max() < 1e-12
    single = plain_zoporax.forward(cfg, weights, toks, dtype=torch.float32).numpy()
    assert row_errors(single, full).max() < 1e-4
    stored = plain_zoporax.forward(cfg, weights, toks, storage=torch.bfloat16).numpy()
    assert 1e-4 < row_errors(stored, full).max() < 0.1
    assert plain_zoporax.greedy(cfg, weights, toks[:5], 3) == plain_zoporax.greedy(cfg, weights, toks[:5], 3)
    folder = make_folder(tmp_path, "only_latent", seed=2)                  # one layer, window 20
    cfg, weights = load(folder)
    toks = tokens(40, cfg["vocab"], 3)
    base = plain_zoporax.forward(cfg, weights, toks).numpy()
    for changed, same in ((10, True), (19, True), (20, False), (39, False)):     # position 39 sees 20..39
        other = list(toks)
        other[changed] = (other[changed] + 1) % cfg["vocab"]
        moved = row_errors(plain_zoporax.forward(cfg, weights, other).numpy()[39:], base[39:]).max()
        assert (moved < 1e-12) == same, (changed, moved)

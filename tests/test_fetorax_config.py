"""Fetorax without a GPU: the typed configuration and its errors, the model as data (which layer writes and
which reads which cache entry, which storage each mixer asks for), the weight table, and the plain
implementation against itself."""
import copy

import pytest
import torch

import plain_fetorax
from fetorax_models import CONFIGS, load, make_folder, row_errors, tokens


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
    assert arch.name == "Fetorax"
    assert _arch(cfg.to_dict())[1] == cfg
    assert cfg.layers[0].rot.factor == 4.0 and cfg.layers[1].rot.factor is None and cfg.layers[1].mlp is None
    spec = arch.describe(cfg)
    assert [(e.layer, e.cache, e.writes_cache) for e in spec.schedule] == \
        [(0, 0, True), (1, 1, True), (2, 2, True), (3, 0, False), (4, 4, True), (5, 4, False)]
    model = Model(spec, Runtime(torch.device("cpu"), torch.float32, 128))
    needs = model.cache_needs()
    assert needs[0] == KVNeed(2, 32, None, 16) and needs[4] == KVNeed(2, 32, None, None)
    assert needs[1] == StateNeed((2, 16, 24)) and needs[2] == StateNeed((3, 25, 41))
    table = model.weight_table()
    assert table["l0.mix.v"].shape == (2 * 16, 64) and table["l0.mix.o"].shape == (64, 6 * 16)
    assert table["l0.mix.sink"].shape == (6,) and table["l0.mix.g"].shape == (6 * 16, 64)
    assert "l3.mix.k" not in table and "l3.mix.v.b" not in table and "l3.mix.q.b" in table
    assert "l1.mlp.up" not in table and "l1.norm2" not in table and table["l2.mlp.up"].shape == (80, 64)
    assert table["l2.mix.i"].shape == (3, 64) and table["l2.mix.f.b"].shape == (3,) and table["l2.mix.norm"].shape == (120,)
    assert model.graph_safe and model.kernel_libraries() == ("recurrent",)


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "earlier"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "attention layer"),
    (lambda c: c["layers"][5]["mixer"].update(kv_from=3), "of its own"),
    (lambda c: c["layers"][3]["mixer"].update(dim=16), "equal"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=4), "multiple"),
    (lambda c: c["layers"][2].update(type="conv"), "not one of"),
    (lambda c: c["layers"][2]["mixer"].pop("gate_cap"), "gate_cap"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "not supported"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.update(layers=[]), "layers"),
])
def test_configuration_errors_name_the_key(change, word):
    from longbow_quarrel_b200.config import ConfigError
    data = copy.deepcopy(CONFIGS["mixed"])
    change(data)
    with pytest.raises(ConfigError, match=word):
        _arch(data)


def test_plain_implementation_agrees_with_itself(tmp_path):
    """A prefix's logits do not depend on what follows (causality of every mixer), float32 stays close to
    float64, and a layer that reads another's keys and values differs from one that would have made its own."""
    folder = make_folder(tmp_path, "mixed", seed=1)
    cfg, weights = load(folder)
    toks = tokens(40, cfg["vocab"], 2)
    full = plain_fetorax.forward(cfg, weights, toks).numpy()
    part = plain_fetorax.forward(cfg, weights, toks[:17]).numpy()
    assert row_errors(part, full[:17]).max() < 1e-12
    single = plain_fetorax.forward(cfg, weights, toks, dtype=torch.float32).numpy()
    assert row_errors(single, full).max() < 1e-4
    stored = plain_fetorax.forward(cfg, weights, toks, storage=torch.bfloat16).numpy()
    assert 1e-4 < row_errors(stored, full).max() < 0.1
    assert float(abs(full).max()) < cfg["logit_softcap"]
    assert plain_fetorax.greedy(cfg, weights, toks[:5], 3) == plain_fetorax.greedy(cfg, weights, toks[:5], 3)

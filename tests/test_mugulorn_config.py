"""Mugulorn's configuration and model description, on the CPU: every size and constant comes from config.json,
layers that read another's cache share its slot, and what cannot run is refused with the key's name."""
import copy

import pytest
import torch

import plain_mugulorn as plain
import tiny_mugulorn as tm
from atom_b200.config.model_config import ConfigError, config_from_dict
from atom_b200.models.model import Model
from atom_b200.models.registry import build_model_spec
from atom_b200.parts.rope import yarn_frequencies
from atom_b200.weights.loader import expected_tensors


@pytest.mark.parametrize("name", list(tm.CONFIGS))
def test_config_round_trip_and_tensor_names(name):
    cfg = config_from_dict(tm.CONFIGS[name])
    assert cfg.architecture == "Mugulorn"
    assert config_from_dict(cfg.to_dict()) == cfg
    model = Model(build_model_spec(cfg))
    want = expected_tensors(model)
    have = tm.random_tensors(tm.CONFIGS[name], 1)
    assert set(want) == set(have)
    for n, (_, _, _, shape, _) in want.items():
        assert tuple(have[n].shape) == tuple(shape), n


def test_cache_slots_windows_and_state():
    cfg = config_from_dict(tm.CONFIGS["A"])
    spec = build_model_spec(cfg)
    assert [(e.layer, e.cache, e.writes_cache) for e in spec.run_order] == [(0, 0, True), (1, 1, True), (2, 0, False), (3, 3, True)]
    needs = Model(spec).cache_needs()
    assert needs[0].kind == "pages" and needs[0].window == 40          # the wider of the owner's 24 and the reader's 40
    assert needs[0].entries[0].shape == (32 + 8,)
    assert needs[1].kind == "state" and {e.name: e.shape for e in needs[1].states} == {"h": (96,), "conv": (2, 96)}
    # a reader without a window makes the cache keep everything
    needs = Model(build_model_spec(config_from_dict(tm.CONFIGS["B"]))).cache_needs()
    assert needs[1].window == 7 and needs[2].window is None and 3 not in needs


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "kv_from"),            # not an attention layer
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "kv_from"),            # itself
    (lambda c: c["layers"][2]["mixer"].update(kv_rank=16), "kv_rank"),           # other sizes than the cache's owner
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), "rot.dims"),      # more than the rotated part holds
    (lambda c: c["layers"][1]["mixer"].update(blocks=5), "blocks"),
    (lambda c: c["layers"][1].update(type="lstm"), "type"),
    (lambda c: c.pop("residual_mult"), "residual_mult"),
    (lambda c: c["layers"][0]["mlp"].update(kind="experts"), "mlp.kind"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
])
def test_refusals_name_the_key(edit, word):
    c = copy.deepcopy(tm.CONFIGS["A"])
    edit(c)
    with pytest.raises(ConfigError, match=word.replace(".", r"\.")):
        config_from_dict(c)


def test_yarn_frequencies_match_the_plain_formula():
    for dims, base, sc in ((8, 10000.0, tm._YARN), (16, 500000.0, {"factor": 8.0, "original": 2048, "fast": 32.0, "slow": 1.0}),
                           (4, 77.0, {"factor": 16.0, "original": 32, "fast": 4.0, "slow": 2.0})):
        f, mag = yarn_frequencies(dims, base, sc["factor"], sc["original"], sc["fast"], sc["slow"])
        pf, pmag = plain.yarn_frequencies(dims, base, sc)
        assert torch.allclose(torch.tensor(f, dtype=torch.float64), pf, rtol=1e-12, atol=0) and abs(mag - pmag) < 1e-12
    # both ends of the ramp are met: the fastest pair keeps its frequency, the slowest is divided by the factor
    f, _ = yarn_frequencies(16, 500000.0, 8.0, 2048, 32.0, 1.0)
    assert f[0] == 1.0 and abs(f[-1] - 500000.0 ** (-14 / 16) / 8.0) < 1e-15

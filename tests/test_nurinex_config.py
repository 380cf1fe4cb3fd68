"""Nurinex on the CPU: configuration (sizes from config.json and from the checkpoint's shapes), the model
spec (layers that run another layer's tensors on a cache of their own), what the cache manager is asked
for, weights by name, and the distance-bias rows as the kernel finds them."""
import os

import pytest
import torch
from safetensors.torch import load_file

import plain_nurinex as plain
import tiny_nurinex as tn
from atom_b200.config import ConfigError, config_from_dict, load_model_config
from atom_b200.models import build_model_spec
from atom_b200.models.model import Model
from atom_b200.parts.mixed_attention import distance_thresholds
from atom_b200.weights import expected_tensors, load_weights


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    out = {}
    for name, cfg in tn.CONFIGS.items():
        d = str(tmp_path_factory.mktemp(f"nurinex_{name}"))
        tn.write_model(cfg, d, tn.SEEDS[name])
        out[name] = d
    return out


@pytest.mark.parametrize("name", list(tn.CONFIGS))
def test_sizes_come_from_config_and_shapes(dirs, name):
    src = tn.CONFIGS[name]
    cfg = load_model_config(dirs[name])
    assert cfg.architecture == "Nurinex" and cfg.vocab == src["vocab"] and cfg.width == src["width"]
    assert cfg.embedding_scale == src["embedding"]["scale"] and cfg.norm_eps == src["norm"]["eps"]
    assert len(cfg.layers) == len(src["layers"])
    for L, e in zip(cfg.layers, src["layers"]):
        lf, rt = e["mixer"]["left"], e["mixer"]["right"]
        assert (L.left.heads, L.left.kv_heads, L.left.dim, L.left.vdim) == (lf["heads"], lf["kv_heads"], lf["dim"], lf["vdim"])
        assert (L.left.scale, L.left.bias_max, L.left.temp_coef, L.left.temp_every) == (
            lf["scale"], lf["bias_max"], lf["q_temp"]["coef"], lf["q_temp"]["every"])
        assert L.left.bias_rows == lf["_rows"] and L.right.decay_rank == rt["_rank"]      # found in the shapes
        assert (L.right.heads, L.right.dim) == (rt["heads"], rt["dim"])
        assert L.ff == (e["mlp"]["ff"] if e["mlp"] else None) and L.weights_of == e.get("weights_of")
    assert cfg.to_dict() == tn.public_config(src)


@pytest.mark.parametrize("name", list(tn.CONFIGS))
def test_spec_runs_shared_layers_on_caches_of_their_own(dirs, name):
    src = tn.CONFIGS[name]
    spec = build_model_spec(load_model_config(dirs[name]))
    own = [i for i, e in enumerate(src["layers"]) if e.get("weights_of") is None]
    assert len(spec.layers) == len(own) and len(spec.run_order) == len(src["layers"])
    assert [e.cache for e in spec.run_order] == list(range(len(src["layers"])))
    for i, e in enumerate(spec.run_order):
        assert own[e.layer] == plain.owner_of(src["layers"], i) and e.writes_cache
    m = Model(spec)
    needs = m.cache_needs()
    assert sorted(needs) == list(range(len(src["layers"])))
    for i, e in enumerate(src["layers"]):
        lf, rt = e["mixer"]["left"], e["mixer"]["right"]
        need = needs[i]
        assert need.kind == "pages" and need.window is None
        assert {x.name: x.shape for x in need.entries} == {"k": (lf["kv_heads"], lf["dim"]), "v": (lf["kv_heads"], lf["vdim"])}
        states = {x.name: (x.shape, x.dtype) for x in need.states}
        assert states["right.wkv"] == ((rt["heads"], rt["dim"], rt["dim"]), "float32")
        assert states["right.shift"][0] == (src["width"],)
    has_ffn = ["ffn" in ls.parts for ls in spec.layers]
    assert has_ffn == [src["layers"][i]["mlp"] is not None for i in own]


@pytest.mark.parametrize("name", list(tn.CONFIGS))
def test_weights_by_name(dirs, name):
    d = dirs[name]
    m = Model(build_model_spec(load_model_config(d)))
    raw = load_file(os.path.join(d, "model.safetensors"))
    assert set(raw) == set(expected_tensors(m))
    w = load_weights(m, d, torch.bfloat16, "cpu")
    assert torch.equal(w["layers.0.mixer.left.qkv.weight"],
                       torch.cat([raw["l0.mix.left.q"], raw["l0.mix.left.k"], raw["l0.mix.left.v"]]))
    assert torch.equal(w["layers.0.mixer.right.mu"].to(torch.bfloat16),
                       torch.stack([raw[f"l0.mix.right.mu.{s}"] for s in "rkvgw"]))
    assert torch.equal(w["layers.0.mixer.left.out"].to(torch.bfloat16), raw["l0.mix.left.out"])
    assert torch.equal(w["lm_head.weight"], raw["head"]) and torch.equal(w["embedding.weight"], raw["embed"])
    w32 = load_weights(m, d, torch.float32, "cpu")
    assert all(t.dtype == torch.float32 for t in w32.values())


def test_configurations_that_are_refused():
    base = tn.public_config(tn.CONFIGS["P"])
    shapes = {"l0.mix.left.rel": (8, 4), "l0.mix.right.w1": (8, 64), "l1.mix.left.rel": (8, 4), "l1.mix.right.w1": (8, 64)}
    config_from_dict(base, shapes)

    def broken(change):
        import copy
        c = copy.deepcopy(base)
        change(c)
        with pytest.raises(ConfigError):
            config_from_dict(c, shapes)

    broken(lambda c: c["layers"][0].__setitem__("type", "serial"))
    broken(lambda c: c["layers"][0]["mixer"]["left"].__setitem__("kv_heads", 3))
    broken(lambda c: c["layers"][2].__setitem__("weights_of", 2))
    broken(lambda c: c["layers"][2].__setitem__("weights_of", 7))
    broken(lambda c: c["layers"][2]["mixer"]["left"].__setitem__("heads", 8))       # other sizes than its owner
    broken(lambda c: c["layers"][0]["mlp"].__setitem__("kind", "routed"))
    broken(lambda c: c["norm"].__setitem__("eps", 0))
    broken(lambda c: c.__delitem__("embedding"))
    with pytest.raises(ConfigError):
        config_from_dict(base, None)            # neither shapes nor the sizes as keys
    import copy
    c = copy.deepcopy(base)
    for L in c["layers"]:
        L["mixer"]["left"]["bias_rows"] = 8
        L["mixer"]["right"]["decay_rank"] = 8
    assert config_from_dict(c, None).layers[0].left.bias_rows == 8


@pytest.mark.parametrize("rows,reach", [(8, 50), (32, 128), (4, 1000), (16, 40.5), (12, 30), (2, 3), (64, 4096), (32, 256),
                                        (6, 3.5), (16, 8.25), (8, 72)])
def test_bias_rows_by_thresholds_equal_the_formula(rows, reach):
    """The kernel finds a distance's row by counting the thresholds at or below it."""
    thr = distance_thresholds(rows, reach)
    half = rows // 2
    assert len(thr) == rows - half - 1 and thr == sorted(thr)
    for n in range(0, int(reach * 3) + 50):
        row = n if n < half else half + sum(1 for t in thr if t <= n)
        assert row == plain.bias_row(n, rows, reach), (n, row)


def test_thresholds_of_a_table_that_reaches_very_far():
    thr = distance_thresholds(32, 1e9)            # (found around their places, not by walking there)
    assert len(thr) == 15 and thr == sorted(thr)
    for t in thr:
        assert plain.bias_row(t, 32, 1e9) == plain.bias_row(t - 1, 32, 1e9) + 1

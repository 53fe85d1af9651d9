"""The Tabedra configuration reader and model description on the CPU: keys, what the tensors' shapes give, the tensor
manifest against the test suite's own list of names and shapes, the run order's cache links, and what is refused."""
import copy

import pytest

import tabedra_models as M
from rustingstrata_b200.config import ConfigError, TabedraConfig, resolve_architecture
from rustingstrata_b200.models.manifest import manifest_for


def spec_of(cfg, rows):
    arch = resolve_architecture(cfg)
    assert arch.name == "Tabedra"
    c = arch.config_class.from_dict(cfg)
    shapes = M.tensor_shapes(cfg, rows)
    return c.resolve_shapes(shapes), arch


@pytest.mark.parametrize("name", sorted(M.CONFIGS))
def test_manifest_matches_the_tests_own_shapes(name):
    cfg, rows = M.CONFIGS[name]
    c, arch = spec_of(cfg, rows)
    assert [L.mixer.bias_rows for L in c.layers] == rows
    # the manifest is computed from a configuration that names the rows itself
    named = copy.deepcopy(cfg)
    for L, r in zip(named["layers"], rows):
        L["mixer"]["bias_rows"] = r
    needs = manifest_for(named)
    want = M.tensor_shapes(cfg, rows)
    assert {k: tuple(v.shape) for k, v in needs.items() if not v.optional} == {k: tuple(v) for k, v in want.items()}


def test_cache_links_and_windows():
    cfg, rows = M.CONFIGS["P"]
    c, arch = spec_of(cfg, rows)
    spec = arch.build_spec(c)
    assert [call.cache for call in spec.order] == [None, None, 0, 0]
    assert spec.n_streams == 3
    # the owner's cache keeps what its widest reader sees
    assert spec.layers[0].parts["mixer"].params["cache_window"] == 52
    assert spec.layers[0].parts["mixer"].params["window"] == 37
    assert spec.layers[1].parts["mixer"].params["cache_window"] is None
    assert spec.layers[3].parts["mixer"].params["kv_projection"] is False
    # a reader without a mask makes the owner keep everything
    cfg2 = copy.deepcopy(cfg)
    del cfg2["layers"][3]["mixer"]["mask"]
    c2, _ = spec_of(cfg2, rows)
    assert arch.build_spec(c2).layers[0].parts["mixer"].params["cache_window"] is None


def test_optional_keys():
    cfg, rows = M.CONFIGS["R"]
    c, arch = spec_of(cfg, rows)
    assert c.streams is None and c.layers[1].mixer.taps == 0 and c.layers[2].mlp is None
    spec = arch.build_spec(c)
    assert spec.n_streams == 1 and not spec.layers[0].block.tensors
    cfg, rows = M.CONFIGS["Q"]
    c, arch = spec_of(cfg, rows)
    assert c.bigram is None and c.streams == 1
    assert arch.build_spec(c).embedding.params["bigram"] is None


@pytest.mark.parametrize("change, text", [
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "earlier layer"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=2), "no keys and values of its own"),
    (lambda c: c["layers"][2]["mixer"].update(heads=12), "head counts"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=4), "not a multiple"),
    (lambda c: c["layers"][0].update(type="recurrent"), "unknown layer type"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "exceeds"),
    (lambda c: c.pop("max_positions"), "max_positions"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_refused_configurations(change, text):
    cfg = copy.deepcopy(M.CONFIGS["P"][0])
    change(cfg)
    with pytest.raises(ConfigError, match=text):
        TabedraConfig.from_dict(cfg)

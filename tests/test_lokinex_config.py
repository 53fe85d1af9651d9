"""Host-side pieces of the Lokinex architecture: configuration, run order, manifest, drawn expert tables, and the
plain implementation's own consistency (no GPU)."""
import numpy as np
import pytest
import torch

import lokinex_models as M
import plain_lokinex as P
from rustingstrata_b200.config import ConfigError, resolve_architecture
from rustingstrata_b200.config.lokinex_config import LokinexConfig
from rustingstrata_b200.models import manifest_for
from rustingstrata_b200.parts.spec import TensorNeed
from rustingstrata_b200.weights.random_init import draw_values


@pytest.mark.parametrize("name", sorted(M.CONFIGS))
def test_manifest_follows_the_configuration(name):
    """The engine asks for exactly the tensors the configuration implies, with their shapes (derived independently)."""
    cfg = M.CONFIGS[name]
    got = {n: tuple(v.shape) for n, v in manifest_for(cfg).items() if not v.optional}
    assert got == M.tensor_shapes(cfg)


def test_architecture_is_found_by_its_key_and_sizes_come_from_the_file():
    cfg = M.CONFIGS["P"]
    arch = resolve_architecture(cfg)
    c = arch.config_class.from_dict(cfg)
    assert isinstance(c, LokinexConfig) and (c.vocab, c.width, c.canon_taps, c.loop) == (211, 96, 3, (1, 3, 3))
    spec = arch.build_spec(c)
    m = spec.layers[1].parts["mixer"].params
    assert (m["n_heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["scale"]) == (3, 16, 8, 24, 40, 24 ** -0.5)
    assert spec.layers[2].parts["mixer_position"].params == {"n_rot": 8, "base": 500.0}
    assert "feed_forward" not in spec.layers[2].parts and "input_conv" in spec.layers[0].parts
    assert "input_conv" not in arch.build_spec(arch.config_class.from_dict(M.CONFIGS["Q"])).layers[0].parts


def test_run_order_of_a_loop():
    """Layers before the loop once, the looped layers ``times`` times, each pass behind a re-entry of its own with its
    pass number, then the rest; every entry of the order is a call of its own (own cache and state)."""
    cfg = M.CONFIGS["P"]
    arch = resolve_architecture(cfg)
    spec = arch.build_spec(arch.config_class.from_dict(cfg))
    kinds = [(spec.layers[c.layer].block.kind, c.layer if c.layer < 4 else spec.layers[c.layer].block.params["index"]) for c in spec.order]
    want = [("sandwich_norm", 0)]
    for t in range(3):
        want += [("stream_reentry", t), ("sandwich_norm", 1), ("sandwich_norm", 2)]
    want += [("sandwich_norm", 3)]
    assert kinds == want and all(c.cache is None for c in spec.order)
    assert [li for li, _, _ in P.run_order(cfg)] == [k[1] for k in kinds if k[0] == "sandwich_norm"]


@pytest.mark.parametrize("bad", [
    lambda c: c.pop("norm"), lambda c: c["layers"][0].update(type="conv"), lambda c: c["loop"].update(stop=9),
    lambda c: c["layers"][1]["mixer"]["rot"].update(dims=9), lambda c: c["layers"][1]["mlp"]["router"].update(top=6),
    lambda c: c["layers"][0]["mixer"].update(blocks=5)])
def test_bad_configurations_are_refused_with_a_sentence(bad):
    import copy
    c = copy.deepcopy(M.CONFIGS["P"])
    bad(c)
    with pytest.raises(ConfigError):
        LokinexConfig.from_dict(c)


def test_drawn_expert_tables_hold_distinct_experts():
    for limit, k in ((16, 2), (5, 5), (7, 1), (9, 4)):
        t = draw_values(3, "l1.mlp.table", TensorNeed((500, k), "choice_table", limit=limit), 0.02, 0.0).reshape(500, k)
        assert t.min() >= 0 and t.max() < limit and all(len(set(r)) == k for r in t.tolist())
        assert len({tuple(r) for r in t.tolist()}) >= min(20, limit)


def test_plain_implementation_is_causal_and_its_convolution_matches_a_sum():
    cfg = M.CONFIGS["P"]
    w = M.draw_weights(cfg, 1)
    toks = np.random.default_rng(0).integers(0, cfg["vocab"], size=30).tolist()
    full = P.forward(toks, w, cfg)
    assert torch.allclose(P.forward(toks[:17], w, cfg), full[:17], atol=1e-12)
    h, k = torch.randn(9, 4, dtype=torch.float64), torch.randn(4, 3, dtype=torch.float64)
    out = P.causal_conv(h, k)
    assert torch.allclose(out[5], k[:, 0] * h[3] + k[:, 1] * h[4] + k[:, 2] * h[5]) and torch.allclose(out[0], k[:, 2] * h[0])

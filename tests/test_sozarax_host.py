"""Host-side tests of the Sozarax design: configuration, the model's description (tensors,
schedule, cache needs) against the plain implementation's own list, and the plain
implementation against itself (a scan cut in two carries its state)."""
import numpy as np
import pytest

from plain import sozarax_plain as P
from test_gpu_sozarax import CFG_A, CFG_B, CFGS


def test_config_round_trip_and_refusals():
    import kllm_b200.models  # noqa: F401  (registers the architectures)
    from kllm_b200.config import ConfigError, parse_config
    for cfg, _ in CFGS.values():
        c = parse_config(cfg)
        assert parse_config(c.to_dict()) == c
        assert c.layer_order() == P.layer_order(cfg)
    no_temp = parse_config(CFG_A).layers[3].mixer
    assert no_temp.q_temp_coef == 0.0 and "q_temp" not in no_temp.to_dict()
    for bad in (dict(CFG_B, loop={"start": 1, "stop": 5, "times": 2}),
                dict(CFG_B, layers=[{"type": "conv", "mixer": {}, "mlp": None}]),
                dict(CFG_B, layers=[{"type": "wkv", "mixer": {"heads": 2, "dim": 8}, "mlp": {"kind": "glu"}}]),
                dict(CFG_B, norm={"eps": 0.0}),
                {k: v for k, v in CFG_B.items() if k != "embedding"}):
        with pytest.raises(ConfigError):
            parse_config(bad)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_model_description(name):
    import torch
    import kllm_b200.models  # noqa: F401
    from kllm_b200.config import build_model_spec, parse_config
    from kllm_b200.parts.model import DecoderModel
    from kllm_b200.parts.spec import PagedKVNeed, StateNeed
    cfg, _ = CFGS[name]
    model = DecoderModel(build_model_spec(parse_config(cfg)), torch.float32, "cpu")
    shapes = P.tensor_shapes(cfg)
    specs = {s.name: s for s in model.tensor_specs()}
    assert set(specs) == set(shapes)
    for n, shape in shapes.items():
        assert specs[n].fits(shape), (n, specs[n].shape, shape)
    order = P.layer_order(cfg)
    assert [c.block for c in model.schedule] == order
    assert [c.cache for c in model.schedule] == list(range(len(order)))      # every run its own cache or state
    for call, need in zip(model.schedule, model.cache_needs()):
        L = cfg["layers"][call.block]
        if L["type"] == "wkv":
            m = L["mixer"]
            floats = m["heads"] * m["dim"] * m["dim"] + cfg["width"]       # the state and the last input row
            assert need == StateNeed((-(-floats // 4) * 4,), "float32")
        else:
            m = L["mixer"]
            assert isinstance(need, PagedKVNeed) and (need.n_kv_heads, need.head_dim, need.value_dim, need.window) == \
                (m["kv_heads"], m["dim"], m["vdim"], None)


def test_cache_manager_with_values_of_another_size():
    import torch
    from kllm_b200.cache.manager import CacheManager
    from kllm_b200.parts.spec import PagedKVNeed, StateNeed
    needs = [PagedKVNeed(2, 16, None, 24), StateNeed((10,)), PagedKVNeed(2, 16, None, 24), PagedKVNeed(2, 16)]
    m = CacheManager(needs, page_size=4, num_pages=6, max_requests=2, dtype=torch.float32)
    assert len(m.groups) == 2 and m.groups[0].slots == [0, 2]
    assert m.bytes_per_page() == (2 * 2 * 4 * (16 + 24) + 2 * 2 * 4 * 16) * 4
    r = m.open()
    m.reserve(r, 9)
    caches = m.layer_caches({0: torch.zeros((1, 3), dtype=torch.int32), 1: torch.zeros((1, 3), dtype=torch.int32)})
    assert tuple(caches[0].k.shape) == (6, 2, 4, 16) and tuple(caches[0].v.shape) == (6, 2, 4, 24)
    assert tuple(caches[3].v.shape) == (6, 2, 4, 16) and caches[1].state.shape == (2, 10)
    caches[0].v.fill_(1.0)
    assert float(caches[0].k.sum()) == 0.0 and float(caches[2].v.sum()) == 0.0     # the views do not overlap
    m.commit(r, 9)
    m.close(r)
    m.audit()


def test_plain_scan_cut_in_two():
    rng = np.random.default_rng(0)
    heads, size, T = 2, 5, 11
    r, k, v = (rng.standard_normal((T, heads * size)) for _ in range(3))
    w, u = rng.uniform(0.2, 0.99, (T, heads * size)), rng.standard_normal(heads * size)
    whole, S = P.wkv_scan(r, k, v, w, u, heads, size)
    a, Sa = P.wkv_scan(r[:4], k[:4], v[:4], w[:4], u, heads, size)
    b, Sb = P.wkv_scan(r[4:], k[4:], v[4:], w[4:], u, heads, size, state=Sa)
    assert np.allclose(np.concatenate([a, b]), whole) and np.allclose(Sb, S)
    # the bonus acts on the current token only: with u = 0 the first token's output is zero
    z, _ = P.wkv_scan(r[:1], k[:1], v[:1], w[:1], 0 * u, heads, size)
    assert np.abs(z).max() == 0.0

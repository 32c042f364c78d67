"""Host-side tests of the Nutizen design: configuration, the model's description (tensors,
schedule, cache needs) against the plain implementation's own list, the cache manager's store
for rows that are keys and values at once, and random weights."""
import numpy as np
import pytest

from plain import nutizen_plain as P
from test_gpu_nutizen import CFG_A, CFG_B, CFGS


def test_config_round_trip_and_refusals():
    import kllm_b200.models  # noqa: F401  (registers the architectures)
    from kllm_b200.config import ConfigError, parse_config
    for cfg, _ in CFGS.values():
        c = parse_config(cfg)
        assert parse_config(c.to_dict()) == c
        assert c.to_dict() == cfg
    layer = CFG_B["layers"][0]

    def with_mixer(**kw):
        return dict(CFG_B, layers=[dict(layer, mixer=dict(layer["mixer"], **kw))])
    for bad in (with_mixer(kv_from=0), with_mixer(mask={"size": 0}), with_mixer(heads=0),
                dict(CFG_B, layers=[dict(layer, type="attention")]),
                dict(CFG_B, layers=[dict(layer, mlp={"kind": "glu"})]),
                dict(CFG_B, layers=[dict(layer, mlp={"kind": "moe", "expert": {"ff": 4, "limit": 0.0},
                                                     "router": {"experts": 2, "top": 1}})]),
                dict(CFG_B, layers=CFG_B["layers"][:2] + [dict(CFG_B["layers"][2],
                                                               mixer=dict(CFG_B["layers"][2]["mixer"], kv_rank=12))]),
                dict(CFG_B, streams=0), dict(CFG_B, norm={"eps": 0.0}),
                {k: v for k, v in CFG_B.items() if k != "embedding"}):
        with pytest.raises(ConfigError):
            parse_config(bad)


@pytest.mark.parametrize("name", sorted(CFGS))
def test_model_description(name):
    import torch
    import kllm_b200.models  # noqa: F401
    from kllm_b200.config import build_model_spec, parse_config
    from kllm_b200.parts.model import DecoderModel
    from kllm_b200.parts.spec import PagedKVNeed
    cfg, _ = CFGS[name]
    model = DecoderModel(build_model_spec(parse_config(cfg)), torch.float32, "cpu")
    shapes = P.tensor_shapes(cfg)
    specs = {s.name: s for s in model.tensor_specs()}
    assert set(specs) == set(shapes)
    for n, (shape, kind) in shapes.items():
        assert specs[n].fits(shape), (n, specs[n].shape, shape)
        assert specs[n].store == ("int32" if kind == "table" else "compute" if kind == "matrix" else "float32"), n
    # a layer with kv_from reads its source's cache slot; that slot keeps the widest window of its readers
    owners = [L["mixer"].get("kv_from", i) for i, L in enumerate(cfg["layers"])]
    slots = {o: k for k, o in enumerate(sorted(set(owners)))}
    assert [(c.block, c.cache, c.writes_cache) for c in model.schedule] == \
        [(i, slots[o], o == i) for i, o in enumerate(owners)]
    for o, need in zip(sorted(set(owners)), model.cache_needs()):
        windows = [(L["mixer"].get("mask") or {}).get("size") for i, L in enumerate(cfg["layers"]) if owners[i] == o]
        widest = None if None in windows else max(windows)
        assert need == PagedKVNeed(1, cfg["layers"][o]["mixer"]["kv_rank"], widest, None, values_are_keys=True)


def test_cache_manager_keeps_one_row_for_keys_and_values():
    import torch
    from kllm_b200.cache.manager import CacheManager
    from kllm_b200.parts.spec import PagedKVNeed
    needs = [PagedKVNeed(1, 24, 40, None, values_are_keys=True), PagedKVNeed(2, 8, None),
             PagedKVNeed(1, 24, 40, None, values_are_keys=True)]
    cm = CacheManager(needs, page_size=4, num_pages=6, max_requests=2, dtype=torch.float32, device="cpu")
    assert len(cm.groups) == 2 and cm.groups[0].slots == [0, 2]
    assert cm.bytes_per_page() == (2 * 1 * 4 * 24 + 1 * 2 * 4 * 16) * 4
    caches = cm.layer_caches({0: None, 1: None})
    assert caches[0].k.data_ptr() == caches[0].v.data_ptr() and tuple(caches[0].k.shape) == (6, 1, 4, 24)
    assert caches[2].k.data_ptr() != caches[0].k.data_ptr() and caches[1].k.data_ptr() != caches[1].v.data_ptr()
    r = cm.open()
    cm.reserve(r, 50 if False else 24)
    cm.commit(r, 24)
    assert sum(p >= 0 for p in r.tables[1]) == 6 and sum(p >= 0 for p in r.tables[0]) == 6
    cm.close(r)
    cm.audit()


def test_random_weights_of_the_design(tmp_path):
    """Random-weights mode fills every tensor of the design, the experts' table with rows of
    different experts, and the loader binds what it wrote."""
    import torch
    from kllm_b200.config import build_model_spec, parse_config
    from kllm_b200.parts.model import DecoderModel
    from kllm_b200.weights import load_weights
    from kllm_b200.weights.random_init import write_random_model
    d = write_random_model(str(tmp_path / "m"), CFG_A, seed=3, dtype=torch.bfloat16)
    model = DecoderModel(build_model_spec(parse_config(CFG_A)), torch.bfloat16, "cpu")
    t = load_weights(d, model.tensor_specs(), torch.bfloat16, "cpu")
    table = t["l1.mlp.table"]
    assert table.dtype == torch.int32 and int(table.min()) >= 0 and int(table.max()) < 4
    assert all(len(set(row.tolist())) == table.shape[1] for row in table)
    assert torch.equal(t["l0.hc1.mix"], torch.eye(2)) and t["l0.hc1.in"].tolist() == [0.5, 0.5]
    model.bind(t)

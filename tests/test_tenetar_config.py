"""Tenetar on the CPU: the reader of config.json, its refusals, the model as data (parts, tensor names, run
order, cache groups), and properties of the plain implementation itself."""
import copy

import numpy as np
import pytest
import torch

import tenetar_helpers as H
import tenetar_plain as P
from x0ne_engine_b200.config import ConfigError, TenetarConfig, config_from_dict, detect
from x0ne_engine_b200.engine.model import CausalLM, step_bytes_of_spec, tensor_needs_of_spec


def test_config_is_read_and_written_back():
    for name, make in H.CONFIGS.items():
        d = make()
        assert detect(d) == "Tenetar"
        c = config_from_dict(d)
        assert isinstance(c, TenetarConfig) and c.to_dict() == d, name
        assert config_from_dict(c.to_dict()) == c


@pytest.mark.parametrize("change,word", [
    (lambda d: d["layers"][0]["mixer"].update(extra=1), "extra"),
    (lambda d: d["layers"][0]["mixer"]["mask"].update(left=1), "left"),
    (lambda d: d["layers"][0]["mixer"].update(heads=5), "multiple"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda d: d["layers"][0].update(type="conv"), "conv"),
    (lambda d: d["layers"][0]["mixer"].update(kv_from=0), "earlier"),
    (lambda d: d["layers"][1]["mixer"].update(kv_from=3), "earlier"),
    (lambda d: d["layers"][3]["mixer"].update(kv_from=1), "no keys"),
    (lambda d: d["layers"][1]["mixer"].update(vdim=13), "differs"),
    (lambda d: d["layers"][1]["mlp"]["router"].update(top=9), "choices"),
    (lambda d: d["layers"][1]["mlp"]["router"]["groups"].update(count=3), "choices"),
    (lambda d: d["layers"][0]["mlp"].update(kind="glu"), "glu"),
    (lambda d: d["norm"].pop("eps"), "eps"),
    (lambda d: d["embedding"].update(scale=0), "scale"),
])
def test_refusals_name_the_key(change, word):
    d = copy.deepcopy(H.CONFIGS["mixed"]())
    change(d)
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    assert word in str(e.value)


def test_spec_parts_names_and_run_order():
    d = H.CONFIGS["mixed"]()
    spec = config_from_dict(d).to_spec()
    assert [l.block for l in spec.layers] == ["sandwich"] * 4
    assert [e.reads_cache_of for e in spec.run_order] == [None, 0, None, 2]
    assert [l.parts["mixer"]["own_kv"] for l in spec.layers] == [True, False, True, False]
    assert "ffn" not in spec.layers[3].parts and spec.layers[1].parts["ffn"].kind == "routed_experts"
    assert spec.layers[0].parts["ffn"].kind == "swiglu" and spec.embedding["scale"] == d["embedding"]["scale"]
    m1 = spec.layers[1].parts["mixer"]
    assert (m1["window"], m1["keep_first"]) == (50, 70)
    assert len(spec.positions) == 2                    # layers with the same rotation share a table
    names = {n.name: tuple(n.shape) for n in tensor_needs_of_spec(spec)}
    t = H.make_tensors(d, 0)
    assert names == {k: tuple(v.shape) for k, v in t.items()}
    assert "l1.mix.k" not in names and "l1.mix.k.norm" not in names and "l3.norm2" not in names
    weights, cache = step_bytes_of_spec(spec)
    # two layers keep keys and values; the readers add nothing
    assert cache == 2 * (2 * (20 + 12)) + 2 * (4 * (16 + 24))


def test_cache_groups_and_readers():
    from x0ne_engine_b200.cache import SequenceCache
    from x0ne_engine_b200.engine.model import cache_need_of_layer
    spec = config_from_dict(H.CONFIGS["mixed"]()).to_spec()
    needs = [cache_need_of_layer(spec.layers[e.layer]) for e in spec.run_order]
    assert all(n.window is None for n in needs)         # kept first keys: the cache holds every position
    cache = SequenceCache(needs, [e.reads_cache_of for e in spec.run_order], 512, 512, torch.float32, "cpu")
    assert len(cache.groups) == 2 and [g.entries for g in cache.groups] == [[0], [2]]
    assert cache.kv_view(1).base == cache.kv_view(0).base and cache.kv_view(3).base == cache.kv_view(2).base
    a = cache.acquire(100)
    b = cache.acquire(65)
    cache.release(a)
    c = cache.acquire(200)                              # pages of the released sequence are used again
    assert set(cache.groups[0].pages_of[c]) & {0, 1} and cache.groups[0].pages_of[b] == [2, 3]


def test_sandwich_block_roles():
    from x0ne_engine_b200.config.spec import LayerSpec
    from x0ne_engine_b200.engine.model import layer_part_classes
    spec = config_from_dict(H.CONFIGS["mixed"]()).to_spec()
    l3 = spec.layers[3]
    assert [r for r, _, _ in layer_part_classes(l3)] == ["mixer_norm", "mixer", "mixer_post_norm"]
    with pytest.raises(ConfigError):
        layer_part_classes(LayerSpec("sandwich", {k: v for k, v in l3.parts.items() if k != "mixer_post_norm"}))


# ---- the plain implementation itself
def test_plain_mask_and_sink():
    m = P.visible(12, 4, 2)
    assert m[11].tolist() == [True, True] + [False] * 6 + [True] * 4
    assert m[3].tolist() == [True] * 4 + [False] * 8 and m[5, 1] and not m[6, 2] and m[6, 3]
    assert P.visible(5, None, 0).tolist() == torch.tril(torch.ones(5, 5, dtype=torch.bool)).tolist()
    s = torch.zeros(1, 1, 3, dtype=torch.float64)
    p = P.sink_softmax(s, torch.ones(1, 3, dtype=torch.bool), torch.tensor([0.0], dtype=torch.float64))
    assert torch.allclose(p, torch.full((1, 1, 3), 0.25, dtype=torch.float64))        # three keys and the sink share the denominator
    assert torch.allclose(P.sink_softmax(s, torch.ones(1, 3, dtype=torch.bool), None), torch.full((1, 1, 3), 1 / 3, dtype=torch.float64))


def test_plain_rotation_is_partial_and_relative():
    x = torch.randn(4, 2, 10, dtype=torch.float64)
    y = P.rotate_half_layout(x, torch.arange(4), 6, 100.0)
    assert torch.equal(y[..., 6:], x[..., 6:]) and torch.equal(y[0], x[0]) and not torch.allclose(y[1, :, :6], x[1, :, :6])
    q, k = torch.randn(1, 1, 6, dtype=torch.float64), torch.randn(1, 1, 6, dtype=torch.float64)
    dots = [float((P.rotate_half_layout(q, torch.tensor([p + 3]), 6, 100.0) * P.rotate_half_layout(k, torch.tensor([p]), 6, 100.0)).sum())
            for p in (0, 5, 40)]
    assert max(dots) - min(dots) < 1e-4


def test_plain_routing_rules():
    n, top = 8, 2
    router = {"experts": 6, "identity": 2, "top": top, "groups": {"count": 4, "keep": 2}}
    w = {"r.router": torch.eye(n), "r.correction": torch.tensor([0., 0., 0., 0., 0., 0., 0., -5.0])}
    z = torch.tensor([[0., 0., 3., 2.9, 0., 0., 2.95, 6.0]], dtype=torch.float64)          # output 7 has the largest score but a large negative correction
    chosen, weights = P.route(z, router, w, "r.")
    s = torch.softmax(z, -1)[0]
    # groups are (0,1) (2,3) (4,5) (6,7): the best two by choice value are (2,3) and (6,7) (through output 6)
    assert sorted(chosen[0].tolist()) == [2, 6]
    assert torch.allclose(weights[0].sort().values, torch.stack([s[2], s[6]]).sort().values)     # plain scores, not renormalized
    assert float(weights.sum()) < 0.2
    # all choice values negative: the groups that are left out still count as lower (as zeros they would win)
    w2 = {"r.router": torch.eye(n), "r.correction": torch.full((n,), -3.0)}
    chosen2, _ = P.route(z, router, w2, "r.")
    assert sorted(chosen2[0].tolist()) == [2, 7]


def test_plain_identity_expert_and_shared_gate():
    cfg = H.CONFIGS["experts_only"]()
    t = H.make_tensors(cfg, 1)
    mlp = cfg["layers"][0]["mlp"]
    h = torch.randn(5, cfg["width"], dtype=torch.float64)
    base = P.moe_ff(h, mlp, t, "l0.mlp.")
    t2 = dict(t)
    t2["l0.mlp.shared.down"] = t["l0.mlp.shared.down"] * 0           # the shared expert vanishes
    closed = P.moe_ff(h, mlp, t2, "l0.mlp.")
    assert not torch.allclose(base, closed)
    no_shared = {**mlp, "shared": None}
    assert torch.allclose(P.moe_ff(h, no_shared, t, "l0.mlp."), closed, atol=1e-9)
    # the gate is one number per row: halving it everywhere (sg = 0) halves the shared part
    t4 = dict(t)
    t4["l0.mlp.shared.sg"] = t["l0.mlp.shared.sg"] * 0
    gate = torch.sigmoid(h @ t["l0.mlp.shared.sg"].double().T)
    assert torch.allclose(P.moe_ff(h, mlp, t4, "l0.mlp.") - closed, (base - closed) * 0.5 / gate, atol=1e-9)
    # a row that chooses only identity experts gets itself times the sum of its weights
    t3 = dict(t2)
    t3["l0.mlp.correction"] = torch.tensor([-9.0] * 6 + [5.0, 5.0])
    only_id = {**mlp, "router": {**mlp["router"], "top": 2, "groups": None}}
    chosen, weights = P.route(h, only_id["router"], t3, "l0.mlp.")
    assert set(chosen.flatten().tolist()) == {6, 7}
    assert torch.allclose(P.moe_ff(h, only_id, t3, "l0.mlp."), weights.sum(-1, keepdim=True) * h, atol=1e-6)

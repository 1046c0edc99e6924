"""Rovurax on the CPU: the configuration reader, the model as data, the checkpoint's tensor names,
the cache geometry its mixers ask for, the rotary frequencies, and the plain implementation's own
properties (which the GPU tests then rest on)."""
import copy
import json
import os

import numpy as np
import pytest
import torch

import rovurax_helpers as H
import rovurax_plain as R


def test_config_is_detected_read_and_written_back():
    from x0ne_engine_b200.config import ConfigError, RovuraxConfig, config_from_dict, detect
    cfg = H.CONFIGS["mixed"]()
    assert detect(cfg) == "Rovurax"
    c = config_from_dict(cfg)
    assert isinstance(c, RovuraxConfig) and c.to_dict() == cfg
    assert config_from_dict(c.to_dict()) == c
    for breaker, words in [
        (lambda d: d["layers"][0].__setitem__("type", "convolution"), "not a mixer"),
        (lambda d: d["layers"][1]["mixer"].__setitem__("window", 4), "does not know"),
        (lambda d: d["layers"][1]["mixer"].__setitem__("kv_heads", 4), "multiple of kv_heads"),
        (lambda d: d["layers"][0]["mixer"]["rot"].__setitem__("dims", 4), "equal rot_dim"),
        (lambda d: d["layers"][1]["mlp"].__setitem__("kind", "experts"), "not implemented"),
        (lambda d: d["layers"][3]["mixer"].__setitem__("vdim", 16), "blends its values"),
        (lambda d: d.pop("norm"), "norm"),
    ]:
        bad = copy.deepcopy(cfg)
        breaker(bad)
        with pytest.raises(ConfigError, match=words):
            config_from_dict(bad)


def test_spec_names_parts_roles_and_tensors():
    from x0ne_engine_b200.config import config_from_dict
    from x0ne_engine_b200.engine.model import cache_need_of_layer, tensor_needs_of_spec
    cfg = H.CONFIGS["mixed"]()
    spec = config_from_dict(cfg).to_spec()
    assert [l.block for l in spec.layers] == ["parallel"] * 5
    assert [l.parts["mixer"].kind for l in spec.layers] == ["latent_attention", "masked_attention", "masked_attention",
                                                           "masked_attention", "latent_attention"]
    # the first blending layer is the source, a layer that does not blend stays out of it
    assert [l.parts["mixer"].get("v_blend") for l in spec.layers[1:4]] == ["source", None, "blend"]
    assert "ffn" not in spec.layers[2].parts and "ffn" in spec.layers[1].parts
    assert set(spec.positions) == {"l0.rot", "l4.rot"} and spec.positions["l4.rot"]["scaling"] is None
    needs = {n.name: n for n in tensor_needs_of_spec(spec)}
    assert set(needs) == set(H.make_tensors(cfg, 0))
    assert needs["l1.mix.vmix"].shape == () and needs["l0.mix.sink"].shape == (3,) and needs["l0.mix.dkv"].shape == (46, 72)
    assert "l2.mix.vmix" not in needs
    # cache: keys and values of their own widths; the latent layer keeps one row and no values
    a, l = cache_need_of_layer(spec.layers[1]), cache_need_of_layer(spec.layers[0])
    assert (a.kv_heads, a.head_dim, a.v_dim) == (2, 20, 12)
    assert (l.kv_heads, l.head_dim, l.v_dim) == (1, 46, 0)


def test_cache_pages_with_other_value_widths():
    from x0ne_engine_b200.cache import SequenceCache
    from x0ne_engine_b200.parts.base import CacheNeed
    needs = [CacheNeed("kv", 2, 20, None, v_dim=12), CacheNeed("kv", 1, 46, None, v_dim=0), CacheNeed("kv", 2, 20, None, v_dim=12),
             CacheNeed("kv", 2, 16, None)]
    c = SequenceCache(needs, [None] * 4, capacity_tokens=256, max_seq_len=256, dtype=torch.float32, device="cpu")
    assert len(c.groups) == 3
    g = c._group_of[0]
    assert g.entries == [0, 2] and g.storage.shape == (2, 4, 2 * 64 * 32)
    v0, v1, v3 = c.kv_view(0), c.kv_view(1), c.kv_view(3)
    assert (v0.page_stride, v0.head_dim, v0.v_dim, v0.value_dim) == (2 * 64 * 32, 20, 12, 12)
    assert (v1.page_stride, v1.head_dim, v1.v_dim, v1.value_dim) == (64 * 46, 46, -1, 0)
    assert (v3.v_dim, v3.value_dim) == (0, 16) and c._group_of[3].storage.shape == (1, 4, 2, 2, 64, 16)
    assert c.bytes_per_token() == (2 * 2 * 32 + 46 + 2 * 2 * 16) * 4
    s = c.acquire(100)
    assert all(len(g.pages_of[s]) == 2 for g in c.groups)
    c.release(s)
    assert c.acquire(0) == s


@pytest.mark.parametrize("dims,base,scaling", [(6, 10000.0, {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}),
                                               (24, 250000.0, {"factor": 6.0, "original": 2048, "fast": 24.0, "slow": 1.5}),
                                               (32, 1e6, {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0}),
                                               (8, 100.0, None)])
def test_rotary_frequencies_against_the_plain_formula(dims, base, scaling):
    from x0ne_engine_b200.parts import yarn_frequencies
    f, mag = yarn_frequencies(dims, base, scaling)
    want_f, want_mag = R.yarn_frequencies(dims, base, scaling)
    assert np.allclose(f, want_f.numpy(), rtol=1e-14, atol=0) and mag == pytest.approx(want_mag, rel=1e-15)
    if scaling:
        plain = base ** (-2.0 * np.arange(dims // 2) / dims)
        assert f[0] == plain[0] or f[0] <= plain[0]
        assert np.all(f <= plain * (1 + 1e-12)) and np.all(f >= plain / scaling["factor"] * (1 - 1e-12))
        assert mag == pytest.approx(0.1 * np.log(scaling["factor"]) + 1.0)


def test_random_folder_from_the_package_initialiser_loads_by_name(tmp_path):
    from x0ne_engine_b200 import RandomInit, write_model_folder
    from x0ne_engine_b200.config import config_from_dict, config_from_folder
    from x0ne_engine_b200.engine.model import tensor_needs_of_spec
    from x0ne_engine_b200.weights import loader, open_folder
    cfg = config_from_dict(H.CONFIGS["even"]())
    write_model_folder(str(tmp_path), cfg, RandomInit(seed=3, norm_jitter=0.1), device="cpu")
    assert config_from_folder(str(tmp_path)) == cfg
    src = open_folder(str(tmp_path))
    loader.check(src, tensor_needs_of_spec(cfg.to_spec()))
    assert src.tensor("l0.mix.vmix").shape == () and src.tensor("l1.mix.sink").shape == (4,)
    src.close()
    with open(os.path.join(str(tmp_path), "config.json")) as f:
        assert json.load(f)["architecture"] == "Rovurax"


# ---- the plain implementation's own properties

def test_plain_chunks_cut_the_past_and_prefixes_do_not_see_the_future():
    d, cfg, t = H.folder("attention_only")
    ids = list(np.random.default_rng(0).integers(0, cfg["vocab"], 40))
    full = H.plain_logits(cfg, t, ids)
    assert np.allclose(H.plain_logits(cfg, t, ids[:23]), full[:23], atol=1e-10)
    # chunk of 9: position 18 starts a chunk, so nothing before it matters to positions 18..26
    other = list(ids)
    other[:18] = [(x + 1) % cfg["vocab"] for x in ids[:18]]
    got = H.plain_logits(cfg, t, other)
    assert np.allclose(got[18:27], full[18:27], atol=1e-10) and not np.allclose(got[17], full[17], atol=1e-3)
    # ... and position 26 sees position 18 (the chunk's first) but 27 does not
    other = list(ids)
    other[18] = (ids[18] + 1) % cfg["vocab"]
    got = H.plain_logits(cfg, t, other)
    assert not np.allclose(got[26], full[26], atol=1e-3) and np.allclose(got[27:], full[27:], atol=1e-10)


def test_plain_sink_gate_and_blend_matter():
    d, cfg, t = H.folder("mixed")
    ids = list(np.random.default_rng(1).integers(0, cfg["vocab"], 30))
    base = H.plain_logits(cfg, t, ids)
    for name, change in [("l0.mix.sink", lambda x: x - 30.0), ("l0.mix.g", lambda x: x * 0.0), ("l3.mix.vmix", lambda x: x * 0.0),
                         ("l4.mix.sink", lambda x: x + 3.0)]:
        t2 = dict(t)
        t2[name] = change(t[name])
        assert np.abs(H.plain_logits(cfg, t2, ids) - base).max() > 1e-3 * np.abs(base).max(), name
    # the source layer's own blend weight is not read
    t2 = dict(t)
    t2["l1.mix.vmix"] = t["l1.mix.vmix"] * 0.0
    assert np.array_equal(H.plain_logits(cfg, t2, ids), base)


def test_plain_clipped_unit_limits():
    h = torch.tensor([[10.0, -10.0, 0.5]], dtype=torch.float64)
    eye = torch.eye(3, dtype=torch.float64)
    y = R.clipped_glu(h, eye, eye, eye, 2.0)[0]
    sig = lambda z: 1.0 / (1.0 + np.exp(-z))
    assert y[0].item() == pytest.approx(2.0 * sig(1.702 * 2.0) * 3.0)          # gate and linear branch both cut at +2
    assert y[1].item() == pytest.approx(-10.0 * sig(-17.02) * (-2.0 + 1.0))    # the gate is not cut from below, the branch is
    assert y[2].item() == pytest.approx(0.5 * sig(0.851) * 1.5)

"""Medirax without a GPU: configuration, registry, tensor names, the order of layers, and the
plain model's mechanisms against properties that follow from their definitions."""
import math

import pytest
import torch

import plain_medirax as pm
import tiny_medirax as tm
from fastmlx_b200 import registry
from fastmlx_b200.config import ConfigError, MediraxConfig
from fastmlx_b200.parts import GatedDeltaMixer, GQAAttention, ParallelBlock
from fastmlx_b200.weights.random_init import random_tensors


def test_registry_finds_the_design_by_its_architecture_key():
    cfg, model = registry.build_model(tm.M1)
    assert isinstance(cfg, MediraxConfig) and cfg.vocab_size == 211
    assert [type(l.mixer) for l in model.layers] == [GQAAttention, GatedDeltaMixer, GatedDeltaMixer, GQAAttention]
    assert all(isinstance(l, ParallelBlock) for l in model.layers)


def test_a_looped_run_is_named_once_per_pass_and_every_pass_has_its_own_cache():
    cfg, model = registry.build_model(tm.M1)
    assert cfg.layer_order() == [0, 1, 2, 1, 2, 3] == pm.layer_order(tm.M1)
    assert [r.layer for r in model.schedule] == [0, 1, 2, 1, 2, 3]
    needs = model.cache_needs()
    assert [kv is not None for kv, _, _ in needs] == [True, False, False, False, False, True]
    assert [st is not None for _, st, _ in needs] == [False, True, True, True, True, False]
    assert all(src is None for _, _, src in needs)
    assert pm.layer_order(tm.M2) == [0, 1, 2] and MediraxConfig.from_dict(tm.M3).layer_order() == [0, 1, 2]


def test_tensor_names_and_shapes():
    _, model = registry.build_model(tm.M1)
    specs = {s.name: s.shape for s in model.weight_specs()}
    assert specs["embed"] == (211, 96) and specs["head"] == (211, 96) and specs["final.norm"] == (96,)
    assert specs["l0.mix.q"] == (96, 96) and specs["l0.mix.q.b"] == (96,) and specs["l0.mix.v"] == (80, 96)
    assert specs["l0.mix.o"] == (96, 160) and specs["l0.mix.o.b"] == (96,) and specs["l0.mlp.down"] == (96, 160)
    assert specs["l1.mix.q.conv"] == (48, 3) and specs["l1.mix.v.conv"] == (160, 3) and specs["l1.mix.b"] == (4, 96)
    assert specs["l1.mix.A_log"] == (4,) and specs["l1.mix.dt_bias"] == (4,) and specs["l1.mix.norm"] == (40,)
    assert "l2.mlp.up" not in specs and specs["l2.norm1"] == (96,)
    assert not any(n.endswith(".weight") or n.endswith(".bias") for n in specs)
    tensors = random_tensors(model, 3)
    model.check_weights(tensors)
    # values of different widths get a page layout of their own; equal widths the common one
    kv0, kv3 = model.cache_needs()[0][0], model.cache_needs()[5][0]
    assert (kv0.head_dim, kv0.value_dim, kv0.window) == (24, 40, 37) and (kv3.head_dim, kv3.value_dim, kv3.window) == (32, 32, 5)


@pytest.mark.parametrize("breakage", [
    lambda c: c["layers"][0].update(type="conv"),
    lambda c: c["layers"][0]["mixer"].update(kv_heads=3),
    lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7),
    lambda c: c["layers"][1]["mixer"].update(conv=0),
    lambda c: c["layers"][1]["mlp"].update(kind="routed"),
    lambda c: c["loop"].update(stop=9),
    lambda c: c.pop("norm"),
    lambda c: c.update(vocab=0),
])
def test_bad_configurations_are_refused(breakage):
    import copy
    c = copy.deepcopy(tm.M1)
    breakage(c)
    with pytest.raises(ConfigError):
        MediraxConfig.from_dict(c)


def test_cache_manager_lays_out_values_of_another_width():
    from fastmlx_b200.cache.manager import CacheManager
    _, model = registry.build_model(tm.M1)
    m = CacheManager(model.cache_needs(), page_size=8, num_pages=6, max_requests=2, dtype=torch.float32)
    assert m.entries[0].kv.shape == (6, 2 * 8 * (24 + 40)) and m.entries[5].kv.shape == (6, 2, 1, 8, 32)
    assert m.entries[1].state.shape == (2, 4 * 40 * 24 + 2 * (2 * 2 * 24 + 4 * 40)) and m.entries[0].state is None
    assert m.entries[2].state.shape == (2, 2 * 16 * 16 + 1 * (2 * 2 * 16 + 2 * 16))
    assert m.bytes_per_token() == 4 * (2 * (24 + 40) + 2 * 32)


# ---- the plain model's mechanisms
def test_plain_rotation_keeps_lengths_and_leaves_the_rest():
    x = torch.randn(5, 3, 12, dtype=torch.float64)
    pos = torch.tensor([0, 1, 7, 100, 1000])
    y = pm.rotate_half_partial(x, pos, 10000.0, 8)
    assert torch.equal(y[..., 8:], x[..., 8:]) and torch.allclose(y[0], x[0])
    assert torch.allclose(y[..., :8].norm(dim=-1), x[..., :8].norm(dim=-1))
    # dimension 0 pairs with dimension 4 and turns by the position itself
    a = 7.0
    assert torch.allclose(y[2, 0, 0], x[2, 0, 0] * math.cos(a) - x[2, 0, 4] * math.sin(a))
    assert torch.allclose(y[2, 0, 4], x[2, 0, 4] * math.cos(a) + x[2, 0, 0] * math.sin(a))


def test_plain_convolution_is_causal_and_its_last_tap_is_the_current_token():
    x = torch.randn(9, 4, dtype=torch.float64)
    w = torch.randn(4, 3, dtype=torch.float64)
    y = pm.causal_conv_silu(x, w)
    assert torch.allclose(y[0], pm.silu(x[0] * w[:, 2]))
    assert torch.allclose(y[5], pm.silu(x[3] * w[:, 0] + x[4] * w[:, 1] + x[5] * w[:, 2]))
    x2 = x.clone()
    x2[6:] += 1.0
    assert torch.equal(pm.causal_conv_silu(x2, w)[:6], y[:6])


def test_plain_delta_rule_stores_and_recalls_a_value():
    """With decay 1 and write strength 1, writing v under a unit key and reading with the same key returns v."""
    D, Dv = 8, 5
    k = pm.unit_vector(torch.randn(D, dtype=torch.float64), 0.0)
    v = torch.randn(Dv, dtype=torch.float64)
    S = torch.zeros(D, Dv, dtype=torch.float64)
    S = S + torch.outer(k, 1.0 * (v - S.T @ k))
    assert torch.allclose(S.T @ k, v)
    # a second write under the same key replaces the value
    v2 = torch.randn(Dv, dtype=torch.float64)
    S = S + torch.outer(k, 1.0 * (v2 - S.T @ k))
    assert torch.allclose(S.T @ k, v2)


def test_plain_forward_is_causal_and_windows_cut_old_tokens():
    _, model = registry.build_model(tm.M2)
    W = {n: t.float() for n, t in random_tensors(model, 5).items()}
    toks = torch.randint(0, 97, (30,), generator=torch.Generator().manual_seed(1)).tolist()
    full = pm.forward(tm.M2, W, toks)
    assert torch.allclose(pm.forward(tm.M2, W, toks[:17]), full[:17], atol=1e-12)

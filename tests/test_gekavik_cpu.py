"""Gekavik without a GPU: configuration, registry, tensor names, the order of layers and passes, the cache
manager's handling of kept first tokens and of pages of latents, the plain model's mechanisms against properties
that follow from their definitions, and the engine's own step function, cache manager and replay program over
plain statements of the kernels against the plain model."""
import copy
import math

import numpy as np
import pytest
import torch

import plain_gekavik as pg
import plain_ops
import tiny
import tiny_gekavik as tg
import traces
from fastmlx_b200 import registry
from fastmlx_b200.cache.manager import CacheManager
from fastmlx_b200.config import ConfigError, GekavikConfig
from fastmlx_b200.parts import GQAAttention, LatentAttention, LoopPass, PagedKVSpec, RoutedExperts, SandwichBlock


def test_registry_finds_the_design_and_builds_its_layers():
    cfg, model = registry.build_model(tg.G1)
    assert isinstance(cfg, GekavikConfig) and cfg.vocab_size == 211 and cfg.residual_mult == 0.45
    blocks = model.layers[:4]
    assert all(isinstance(b, SandwichBlock) for b in blocks)
    assert [type(b.mixer) for b in blocks] == [GQAAttention, LatentAttention, GQAAttention, LatentAttention]
    assert [type(b.ffn) for b in blocks] == [RoutedExperts, RoutedExperts, type(None), RoutedExperts]
    assert all(isinstance(p, LoopPass) for p in model.layers[4:]) and len(model.layers) == 6


def test_every_pass_of_a_loop_has_its_entry_and_its_own_cache():
    cfg, model = registry.build_model(tg.G1)
    assert cfg.layer_passes() == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)] == pg.layer_passes(tg.G1)
    assert [r.layer for r in model.schedule] == [0, 4, 1, 2, 5, 1, 2, 3]
    needs = model.cache_needs()
    assert [kv is not None for kv, _, _ in needs] == [True, False, True, True, False, True, True, True]
    assert all(st is None and src is None for _, st, src in needs)
    # a loop from the first layer on, three passes; no loop; a loop of one pass
    assert [r.layer for r in registry.build_model(tg.G3)[1].schedule] == [3, 0, 1, 4, 0, 1, 5, 0, 1, 2]
    assert [r.layer for r in registry.build_model(tg.G2)[1].schedule] == [0, 1, 2]
    assert [r.layer for r in registry.build_model(tg.G4)[1].schedule] == [0, 2, 1]


def test_tensor_names_shapes_and_cache_needs():
    _, model = registry.build_model(tg.G1)
    specs = {s.name: s.shape for s in model.weight_specs()}
    assert specs["embed"] == (211, 96) and specs["head"] == (211, 96) and specs["final.norm.alpha"] == ()
    assert specs["loop.in"] == (96, 192) and specs["loop.step"] == (2, 96)
    assert specs["l0.mix.q"] == (96, 96) and specs["l0.mix.q.b"] == (96,) and specs["l0.mix.v"] == (80, 96)
    assert specs["l0.mix.q.norm"] == (24,) and specs["l0.mix.g"] == (160, 96) and specs["l0.mix.o"] == (96, 160)
    assert "l0.mix.o.b" not in specs and "l0.mix.g.b" not in specs
    assert specs["l1.mix.dq"] == (40, 96) and specs["l1.mix.dq.norm"] == (40,) and specs["l1.mix.uq"] == (48, 40)
    assert specs["l1.mix.dkv"] == (48, 96) and specs["l1.mix.uk"] == (48, 48) and specs["l1.mix.uv"] == (72, 48)
    assert specs["l1.mix.g"] == (3, 96) and specs["l1.mix.o"] == (96, 72)
    assert specs["l0.mlp.router"] == (8, 96) and specs["l0.mlp.e7.down"] == (96, 48) and specs["l0.mlp.shared.up"] == (32, 96)
    assert "l1.mlp.shared.gate" not in specs and "l2.mlp.router" not in specs and "l2.norm2" not in specs
    assert specs["l2.norm1b.b"] == (96,) and specs["l3.norm2b.alpha"] == ()
    tensors = tg.lively_tensors(tg.G1, 3)
    model.check_weights(tensors)
    # a checkpoint that stores a second pair of norms for a layer without a feed-forward is read all the same
    extra = dict(tensors, **{"l2.norm2": torch.ones(96), "l2.norm2.b": torch.zeros(96), "l2.norm2b.alpha": torch.ones(())})
    model.check_weights(extra)
    needs = model.cache_needs()
    assert needs[0][0] == PagedKVSpec(2, 24, 37, 40, 3, False)
    assert needs[2][0] == PagedKVSpec(1, 48, 21, 0, 0, True) and needs[7][0] == PagedKVSpec(1, 64, 0, 0, 0, True)


@pytest.mark.parametrize("breakage", [
    lambda c: c["layers"][0].update(type="delta"),
    lambda c: c["layers"][0]["mixer"].update(kv_heads=3),
    lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7),
    lambda c: c["layers"][0]["mlp"]["router"].update(top=9),
    lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=3),
    lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(keep=3),
    lambda c: c["layers"][1]["mlp"].update(kind="dense"),
    lambda c: c["layers"][1]["mixer"].pop("kv_rank"),
    lambda c: c["loop"].update(stop=9),
    lambda c: c.pop("norm"),
    lambda c: c.update(vocab=0),
])
def test_bad_configurations_are_refused(breakage):
    c = copy.deepcopy(tg.G1)
    breakage(c)
    with pytest.raises(ConfigError):
        GekavikConfig.from_dict(c)


# ---- the cache manager
def test_pages_of_kept_first_tokens_stay_while_the_window_gives_the_others_back():
    spec = PagedKVSpec(1, 8, window=20, keep_first=19)              # 19 kept tokens: the first two pages of 16
    m = CacheManager([(spec, None, None)], page_size=16, num_pages=8, max_requests=2, dtype=torch.float32)
    r = m.add_request("a")
    for n in (10, 30, 1, 1, 60, 1):
        m.reserve(r, n)
        m.commit(r)
        m.check()
    bt = r.tables[0]
    assert r.length == 103 and bt.kept == 2 and bt.pages[0] >= 0 and bt.pages[1] >= 0
    # position 103 sees keys 84..103 (page 5 on) and 0..18: pages 2, 3, 4 are back in the pool
    assert bt.pages[2:5] == [-1, -1, -1] and all(p >= 0 for p in bt.pages[5:])
    assert m.groups[0].pool.used_pages == 2 + len(bt.pages) - 5
    m.free("a")
    m.check()
    assert m.groups[0].pool.used_pages == 0
    # a pool that holds the window, the kept pages and a portion serves a long request
    assert m.holds_alone(10000, 16) == 0


def test_a_window_shorter_than_the_kept_tokens_page_and_a_short_request():
    spec = PagedKVSpec(2, 4, window=3, keep_first=1)
    m = CacheManager([(spec, None, None)], page_size=4, num_pages=4, max_requests=1, dtype=torch.float32)
    r = m.add_request("a")
    for _ in range(30):
        m.reserve(r, 1)
        m.commit(r)
        m.check()
    assert r.tables[0].pages[0] >= 0 and m.groups[0].pool.used_pages <= 3


def test_pages_of_latents_hold_keys_only():
    _, model = registry.build_model(tg.G1)
    m = CacheManager(model.cache_needs(), page_size=8, num_pages=6, max_requests=2, dtype=torch.float32)
    assert m.entries[0].kv.shape == (6, 2 * 8 * (24 + 40)) and m.entries[2].kv.shape == (6, 1, 1, 8, 48)
    assert m.entries[1].kv is None and m.entries[3].kv.shape == (6, 2, 2, 8, 32)
    # two passes of the loop: entries 2 and 5 are the same layer with pages of their own
    assert m.entries[2].kv.data_ptr() != m.entries[5].kv.data_ptr()
    assert m.bytes_per_token() == 4 * (2 * (24 + 40) + 2 * 48 + 2 * (2 * 2 * 32) + 64)


# ---- the plain model's mechanisms
def test_plain_rotation_turns_neighbouring_pairs_and_leaves_the_rest():
    x = torch.randn(5, 3, 12, dtype=torch.float64)
    pos = torch.tensor([0, 1, 7, 100, 1000])
    y = pg.rotate_pairs(x, pos, 10000.0, 8)
    assert torch.equal(y[..., 8:], x[..., 8:]) and torch.allclose(y[0], x[0])
    assert torch.allclose(y[..., :8].norm(dim=-1), x[..., :8].norm(dim=-1))
    a = 7.0 * 10000.0 ** (-2.0 / 8)                 # pair 1 = dimensions (2, 3)
    assert torch.allclose(y[2, 0, 2], x[2, 0, 2] * math.cos(a) - x[2, 0, 3] * math.sin(a))
    assert torch.allclose(y[2, 0, 3], x[2, 0, 3] * math.cos(a) + x[2, 0, 2] * math.sin(a))
    # the score of a rotated pair depends on the distance alone
    q, k = torch.randn(1, 1, 8, dtype=torch.float64), torch.randn(1, 1, 8, dtype=torch.float64)
    s = [float((pg.rotate_pairs(q, torch.tensor([p + 9]), 50.0, 8) * pg.rotate_pairs(k, torch.tensor([p]), 50.0, 8)).sum())
         for p in (0, 31)]
    assert abs(s[0] - s[1]) < 1e-9


def test_plain_mask_keeps_the_window_and_the_first_tokens():
    seen = pg.visible(12, size=4, keep_first=2)
    assert seen[9].tolist() == [True, True, False, False, False, False, True, True, True, True, False, False]
    assert seen[3].tolist() == [True] * 4 + [False] * 8 and seen[4].tolist()[:6] == [True, True, True, True, True, False]
    assert torch.equal(pg.visible(7), torch.tril(torch.ones(7, 7, dtype=torch.bool)))
    assert pg.visible(9, size=3)[8].tolist() == [False] * 6 + [True] * 3


def test_plain_router_chooses_within_the_best_groups_and_does_not_renormalise():
    z = torch.tensor([[0.0, 5.0, 1.0, 1.1, 4.0, 0.2, 3.0, 3.1]], dtype=torch.float64)
    s = torch.softmax(z, -1)
    w = pg.route(z, 3, 4, 2)                       # groups (0,1) (2,3) (4,5) (6,7): the best two are the first and the third
    assert torch.nonzero(w[0]).flatten().tolist() == [1, 4, 5] and torch.allclose(w[0, [1, 4, 5]], s[0, [1, 4, 5]])
    assert float(w.sum()) < 1.0
    assert torch.nonzero(pg.route(z, 3, 1, 1)[0]).flatten().tolist() == [1, 4, 7]
    assert torch.nonzero(pg.route(z, 3, 4, 4)[0]).flatten().tolist() == [1, 4, 7]
    assert torch.equal(plain_ops.moe_route(z.float(), 3, 4, 2) > 0, w > 0)


def test_plain_expert_clamps_before_the_activation():
    h = torch.tensor([[1.0, -2.0]], dtype=torch.float64)
    gate = torch.tensor([[3.0, 0.0], [-4.0, 0.0]], dtype=torch.float64)
    up = torch.tensor([[0.0, 2.0], [0.0, -0.1]], dtype=torch.float64)
    down = torch.eye(2, dtype=torch.float64)
    y = pg.expert(h, gate, up, down, 1.5)          # gates 3 -> 1.5 and -4 stays; ups -4 -> -1.5 and 0.2
    g0, g1 = 1.5, -4.0
    want = [g0 / (1 + math.exp(-1.702 * g0)) * (-1.5 + 1), g1 / (1 + math.exp(-1.702 * g1)) * (0.2 + 1)]
    assert torch.allclose(y[0], torch.tensor(want, dtype=torch.float64))


def test_plain_latent_attention_caches_what_is_enough():
    """Keys and values are functions of the latent alone: carrying the query into the latent's space gives the
    same scores, and reading the values out after the weighted sum the same outputs."""
    T, H, D, Dv, R = 6, 2, 4, 3, 5
    c = torch.randn(T, R, dtype=torch.float64)
    q = torch.randn(T, H, D, dtype=torch.float64)
    uk, uv = torch.randn(H * D, R, dtype=torch.float64), torch.randn(H * Dv, R, dtype=torch.float64)
    seen = pg.visible(T, 4)
    for h in range(H):
        direct = pg.softmax_attention(q[:, h], (c @ uk.T).view(T, H, D)[:, h], (c @ uv.T).view(T, H, Dv)[:, h], 0.3, seen)
        q_lat = q[:, h] @ uk.view(H, D, R)[h]
        via = pg.softmax_attention(q_lat, c, c, 0.3, seen) @ uv.view(H, Dv, R)[h].T
        assert torch.allclose(direct, via)


def test_plain_forward_is_causal():
    W = {n: t.double() for n, t in tg.lively_tensors(tg.G2, 5).items()}
    toks = tiny.rand_tokens(30, 97, 1)
    full = pg.forward(tg.G2, W, toks)
    assert torch.allclose(pg.forward(tg.G2, W, toks[:17]), full[:17], atol=1e-12)


# ---- the engine over plain statements of the kernels
LENS = {"G1": [1, 2, 9, 45, 58], "G2": [3, 50, 75], "G3": [5, 40], "G4": [4, 41, 23]}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("gekavik_cpu")
    out = {}
    for name, cfg in tg.CONFIGS.items():
        d = tg.make_model_dir(root, cfg, seed=11)
        W = tiny.load_plain_weights(d)
        prompts = {f"r{i}": tiny.rand_tokens(n, cfg["vocab"], 500 + i) for i, n in enumerate(LENS[name])}
        out[name] = (d, prompts, {r: pg.forward(cfg, W, t) for r, t in prompts.items()})
    return out


@pytest.mark.parametrize("name", ["G1", "G2", "G3", "G4"])
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed"])
def test_engine_over_plain_kernels_matches_the_plain_model(models, name, cut):
    from fastmlx_b200.engine.replay import Replayer
    d, prompts, ref = models[name]
    steps = {"whole": traces.whole, "tail": lambda p: traces.tail_decoded(p, tail=12), "portions": traces.portions,
             "mixed": lambda p: traces.mixed(p, max_live=2)}[cut](prompts)
    rp = Replayer(d, "float32", 160, page_size=8, device="cpu", kernels=plain_ops, max_live=2)
    outs = []
    for st in steps:
        outs.append(rp.step(st))
        rp.manager.check()
    assert not rp.manager.requests and all(g.pool.used_pages == 0 for g in rp.manager.groups)
    rows = traces.collect(steps, outs)
    for rid, toks in prompts.items():
        got = torch.from_numpy(np.stack([rows[rid][i] for i in range(len(toks))])).double()
        err = (got - ref[rid]).abs().max() / ref[rid].abs().max()
        assert err < 2e-5, (rid, float(err))

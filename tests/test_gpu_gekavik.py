"""Gekavik on the GPU against the plain model of tests/plain_gekavik.py: each mechanism's kernels alone, whole
prompts against decoding token by token, portions down to two tokens, mixed batches over pools and slots that are
used again, keys made to stand out just inside and just outside the window and the kept first tokens, far keys, long
decoding, and greedy generation through the engine."""
import math

import numpy as np
import pytest
import torch

import plain_gekavik as pg
import plain_ops
import tiny
import tiny_gekavik as tg
import traces

pytestmark = pytest.mark.gpu

# Largest |difference| as a fraction of the largest |logit| of the plain model (float64).  32-bit: float32 sums
# against float64.  bfloat16: weights are bfloat16 in both; the engine rounds activations.
TOL = {"float32": 2e-5, "bfloat16": 4e-2}
CASES = {
    "G1": dict(lens=[1, 2, 7, 45, 38, 100, 39, 76, 131], page=16, max_tokens=448),
    "G2": dict(lens=[3, 17, 72, 140, 71, 33, 90], page=16, max_tokens=384),
    "G3": dict(lens=[5, 64, 33, 97, 20, 50, 70], page=32, max_tokens=384),
    "G4": dict(lens=[4, 40, 23, 66, 35, 80], page=16, max_tokens=256),
}
DEV = "cuda"
# A router that takes bfloat16 inputs sees its logits moved by a few hundredths; where the plain model's own choice
# of experts is decided by less (in some layer), either choice is right, and the position is not compared in bfloat16.
CLOSE_CALL = 0.15
CLOSE = {}


def _prompts(name):
    return {f"r{i}": tiny.rand_tokens(n, tg.CONFIGS[name]["vocab"], 300 + i) for i, n in enumerate(CASES[name]["lens"])}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("gekavik")
    out = {}
    for name, cfg in tg.CONFIGS.items():
        d = tg.make_model_dir(root, cfg, seed=23)
        W = tiny.load_plain_weights(d)
        prompts = _prompts(name)
        ref = {}
        for r, t in prompts.items():
            margins = []
            ref[r] = pg.forward(cfg, W, t, margins=margins)
            CLOSE[(name, r)] = torch.stack(margins).min(0).values < CLOSE_CALL
        out[name] = (d, W, prompts, ref)
    return out


def _run(model_dir, dtype, steps, max_tokens, page, max_live=4):
    from fastmlx_b200.engine.replay import Replayer
    rp = Replayer(model_dir, dtype, max_tokens, page_size=page, max_live=max_live)
    outs = []
    for st in steps:
        outs.append(rp.step(st))
        rp.manager.check()
    assert not rp.manager.requests and all(g.pool.used_pages == 0 for g in rp.manager.groups)
    return outs, rp


def _compare(steps, outs, prompts, ref, tol, skip=None):
    rows = traces.collect(steps, outs)
    for rid, toks in prompts.items():
        assert sorted(rows[rid]) == list(range(len(toks)))
        got = torch.from_numpy(np.stack([rows[rid][i] for i in range(len(toks))])).double()
        err = (got - ref[rid]).abs().max(dim=1).values / ref[rid].abs().max().item()
        if skip is not None:
            assert skip[rid].double().mean().item() < 0.5 or len(toks) < 8, "too few positions are compared"
            err = err.masked_fill(skip[rid], 0.0)
        bad = torch.nonzero(err > tol)
        assert bad.numel() == 0, (f"request {rid}: first wrong position {int(bad[0])} of {len(toks)}, "
                                  f"error {err[int(bad[0])].item():.3e} (allowed {tol:.1e})")


CUTS = {"whole": traces.whole, "tail": traces.tail_decoded, "portions": traces.portions, "mixed": traces.mixed,
        "ones": lambda p: traces.tail_decoded(p, tail=10 ** 6)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["G1", "G2", "G3", "G4"])
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed", "ones"])
def test_replay(models, name, dtype, cut):
    d, W, prompts, ref = models[name]
    case = CASES[name]
    steps = CUTS[cut](prompts)
    outs, rp = _run(d, dtype, steps, case["max_tokens"], case["page"])
    _compare(steps, outs, prompts, ref, TOL[dtype], {r: CLOSE[(name, r)] for r in prompts} if dtype == "bfloat16" else None)
    if cut == "mixed":
        need = sum(-(-len(t) // case["page"]) for t in prompts.values())
        assert all(need > g.pool.num_pages for g in rp.manager.groups), "the pool is too large for pages to be used again"
        assert len(prompts) > rp.manager.max_requests, "too many slots for one to be used again"


@pytest.mark.parametrize("name", ["G1", "G2"])
def test_cuts_agree_in_32_bit_to_the_bit(models, name):
    """No sum's order depends on the cut, the batch or the pages: in 32-bit the logits are equal."""
    d, W, prompts, ref = models[name]
    case = CASES[name]
    base_steps = traces.whole(prompts)
    base = traces.collect(base_steps, _run(d, "float32", base_steps, case["max_tokens"], case["page"])[0])
    for cut in ("tail", "portions", "mixed"):
        steps = CUTS[cut](prompts)
        rows = traces.collect(steps, _run(d, "float32", steps, case["max_tokens"], case["page"])[0])
        for rid in prompts:
            for i, row in rows[rid].items():
                assert np.array_equal(row, base[rid][i]), (cut, rid, i, np.abs(row - base[rid][i]).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_moves_the_windows_over_decoded_tokens(models, dtype):
    """130 tokens decoded one by one behind a short prompt: the windows of 70 and 40 pass over decoded tokens, the 19
    kept first tokens stay in sight, pages behind the windows go back to the pool on the way."""
    d, W, prompts, ref = models["G2"]
    sub = {"r3": prompts["r3"]}
    steps = traces.tail_decoded(sub, tail=130)
    outs, _ = _run(d, dtype, steps, 256, 16)
    _compare(steps, outs, sub, ref, TOL[dtype], {"r3": CLOSE[("G2", "r3")]} if dtype == "bfloat16" else None)


@pytest.mark.parametrize("name", ["G2", "G3"])
def test_long_portions_read_keys_and_values_out_of_the_latents(models, name):
    """Portions of 128 tokens and more take latent attention's other form in bfloat16 (keys and values of the tokens in
    sight read out of the cached latents, for the step): whole prompts, two long portions, a long portion behind a
    short one, and a long portion beside single tokens of another request, against the plain model."""
    d, W, _, _ = models[name]
    cfg = tg.CONFIGS[name]
    prompts = {"a": tiny.rand_tokens(300, cfg["vocab"], 71), "b": tiny.rand_tokens(200, cfg["vocab"], 72)}
    ref, skip = {}, {}
    for r, t in prompts.items():
        margins = []
        ref[r] = pg.forward(cfg, W, t, margins=margins)
        skip[r] = torch.stack(margins).min(0).values < CLOSE_CALL
    a, b = prompts["a"], prompts["b"]

    def entry(rid, toks):
        return {"id": rid, "tokens": toks, "want": list(range(len(toks)))}

    schedules = {
        "whole": traces.whole(prompts),
        "portions": [{"step": 0, "entries": [entry("a", a[:130])], "end": []}, {"step": 1, "entries": [entry("a", a[130:])], "end": ["a"]},
                     {"step": 2, "entries": [entry("b", b[:7])], "end": []}, {"step": 3, "entries": [entry("b", b[7:])], "end": ["b"]}],
        "mixed": [{"step": 0, "entries": [entry("b", b[:190])], "end": []}] +
                 [{"step": 1 + i, "entries": [entry("b", [b[190 + i]]), entry("a", a[150 * i:150 * (i + 1)])], "end": ["a"] if i == 1 else []}
                  for i in range(2)] +
                 [{"step": 3 + i, "entries": [entry("b", [b[192 + i]])], "end": ["b"] if i == 7 else []} for i in range(8)],
    }
    for cut, steps in schedules.items():
        outs, _ = _run(d, "bfloat16", steps, 640, 16)
        _compare(steps, outs, prompts, ref, TOL["bfloat16"], skip)


@pytest.mark.parametrize("seed", [1, 2, 4, 5, 6, 7, 9])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_of_configurations_drawn_from_a_seed(tmp_path, seed, dtype):
    """Sizes, counts, constants and the order of layers drawn at random: whole prompts and mixed batches against the plain model."""
    cfg = tg.random_config(seed)
    d = tg.make_model_dir(tmp_path, cfg, seed=seed)
    W = tiny.load_plain_weights(d)
    prompts = {f"r{i}": tiny.rand_tokens(n, cfg["vocab"], 40 * seed + i) for i, n in enumerate([2, 35, 150, 64, 101])}
    ref, skip = {}, {}
    for r, t in prompts.items():
        margins = []
        ref[r] = pg.forward(cfg, W, t, margins=margins)
        skip[r] = torch.stack(margins).min(0).values < CLOSE_CALL if margins else torch.zeros(len(t), dtype=torch.bool)
    for cut in ("whole", "mixed"):
        steps = CUTS[cut](prompts)
        outs, _ = _run(d, dtype, steps, 512, 16)
        _compare(steps, outs, prompts, ref, TOL[dtype], skip if dtype == "bfloat16" else None)


@pytest.mark.parametrize("name", ["G1", "G3", "G5"])
def test_replay_with_grouped_expert_products(tmp_path, monkeypatch, name):
    """The same models with the routed experts' grouped products forced on (they are chosen by size): `mma.sync` tiles for
    steps below 128 tokens and for experts of any width, the tcgen05 kernel for longer portions over experts in blocks of 128
    (G5); whole prompts, portions, and mixed batches, in bfloat16 against the plain model."""
    from fastmlx_b200.parts import RoutedExperts
    monkeypatch.setattr(RoutedExperts, "SPARSE_MIN_BYTES", 0)
    cfg = getattr(tg, name)
    d = tg.make_model_dir(tmp_path, cfg, seed=31)
    W = tiny.load_plain_weights(d)
    prompts = {f"r{i}": tiny.rand_tokens(n, cfg["vocab"], 800 + i) for i, n in enumerate([3, 40, 200, 77, 150])}
    ref, skip = {}, {}
    for r, t in prompts.items():
        margins = []
        ref[r] = pg.forward(cfg, W, t, margins=margins)
        skip[r] = torch.stack(margins).min(0).values < CLOSE_CALL
    for cut in ("whole", "portions", "mixed"):
        steps = CUTS[cut](prompts)
        outs, rp = _run(d, "bfloat16", steps, 640, 16)
        assert any(b.ffn is not None and b.ffn.sparse for b in rp.model.layers if hasattr(b, "ffn"))      # where experts outnumber twice the chosen
        _compare(steps, outs, prompts, ref, TOL["bfloat16"], skip)


# ----------------------------------------------------------------------------- kernels alone
def _k():
    from fastmlx_b200 import kernels
    return kernels


@pytest.mark.parametrize("y_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_dynamic_tanh_step(y_dtype, out_dtype):
    """Norm behind a sublayer, scaled sum into the stream, a vector, norm in front of the next: every combination
    that a block, a loop's entry and the final norm use, against the plain statement."""
    k = _k()
    g = torch.Generator().manual_seed(3)
    T, n = 9, 50
    y = (torch.randn(T, n + 6, generator=g) * 2).to(y_dtype)
    res = torch.randn(T, n, generator=g) * 3
    post = (0.8, torch.randn(n, generator=g), torch.randn(n, generator=g))
    pre = (1.3, torch.randn(n, generator=g), torch.randn(n, generator=g))
    add = torch.randn(n, generator=g)
    tol = 1e-5 if out_dtype == torch.float32 else 1e-2

    def dev(t):
        return None if t is None or t is False else tuple(x.to(DEV) if torch.is_tensor(x) else x for x in t)

    for p_, q_, a_, r_ in [(post, pre, None, res), (None, pre, None, None), (None, pre, add, None), (post, None, None, res),
                           (post, False, add, res)]:
        want_o, want_r = plain_ops.dyt_step(y[:, 3:3 + n], p_, 0.3, a_, None if r_ is None else r_.clone(), q_, out_dtype)
        wide = torch.zeros(T, n + 10, dtype=out_dtype, device=DEV)
        got_o, got_r = k.dyt_step(y.to(DEV)[:, 3:3 + n], dev(p_), 0.3, None if a_ is None else a_.to(DEV),
                                  None if r_ is None else r_.clone().to(DEV), dev(q_), out_dtype,
                                  out=None if q_ is False else wide[:, 4:4 + n])
        assert torch.allclose(got_r.cpu(), want_r, atol=1e-5, rtol=1e-5)
        if q_ is not False:
            assert torch.allclose(got_o.cpu().double(), want_o.double(), atol=tol, rtol=tol)
            assert wide[:, :4].abs().max().item() == 0 and wide[:, 4 + n:].abs().max().item() == 0


def test_norm_of_a_slice_into_rows_named_by_a_map_and_gates():
    k = _k()
    g = torch.Generator().manual_seed(4)
    T, n = 11, 36
    x = torch.randn(T, n + 20, generator=g) * 2
    w = torch.randn(n, generator=g)
    want = plain_ops.rmsnorm_rows(x[:, 7:7 + n], w, 1e-4, out_dtype=torch.float32)
    got = k.rmsnorm_rows(x.to(DEV)[:, 7:7 + n], w.to(DEV), 1e-4, out_dtype=torch.float32)
    assert torch.allclose(got.cpu(), want, atol=1e-5, rtol=1e-5)
    rows = torch.zeros(40, n, dtype=torch.bfloat16, device=DEV)
    row_map = torch.tensor([5, 0, -1, 39, 17, 2, 3, 4, 6, 8, 9], dtype=torch.int64)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    k.rmsnorm_rows(x.to(DEV)[:, 7:7 + n], w.to(DEV), 1e-4, out=rows, row_map=row_map.to(DEV), status=status)
    for t, r in enumerate(row_map.tolist()):
        if r >= 0:
            assert torch.allclose(rows[r].cpu().float(), want[t], atol=2e-2, rtol=2e-2)
    assert rows[1].abs().max().item() == 0 and status.tolist()[0] == 0
    # a row beyond the cache leaves a code and writes nothing
    k.rmsnorm_rows(x.to(DEV)[:1, 7:7 + n], w.to(DEV), 1e-4, out=rows, row_map=torch.tensor([40], device=DEV), status=status)
    assert status.tolist()[0] == 2
    for group, dt in ((1, torch.float32), (12, torch.bfloat16), (12, torch.float32)):
        o = (torch.randn(T, 36, generator=g) * 2).to(dt)
        gate = torch.randn(T, 36 // group + 3, generator=g)
        want = plain_ops.sigmoid_gate(o.clone(), gate[:, 1:1 + 36 // group], group)
        got = k.sigmoid_gate(o.to(DEV), gate.to(DEV)[:, 1:1 + 36 // group], group)
        assert torch.allclose(got.cpu().float(), want.float(), atol=1e-2 if dt == torch.bfloat16 else 1e-6)


@pytest.mark.parametrize("E,top,groups,keep", [(8, 2, 4, 2), (12, 4, 4, 3), (6, 3, 2, 1), (5, 2, 1, 1), (64, 6, 8, 3), (96, 8, 1, 1),
                                                 (9, 2, 3, 3), (4, 4, 2, 2)])
def test_router_against_the_plain_choice(E, top, groups, keep):
    k = _k()
    g = torch.Generator().manual_seed(E * 10 + top)
    z = torch.randn(70, E, generator=g) * 3
    z[3] = 0.0                                   # every score equal: the lowest indices of the first groups win
    z[4, :] = torch.arange(E, 0, -1).float()     # and a row that is sorted already
    want, want_ids = plain_ops.moe_route(z, top, groups, keep, want_chosen=True)
    got, ids = k.moe_route(z.to(DEV), top, groups, keep, want_chosen=True)
    assert torch.equal(got.cpu() > 0, want > 0) and torch.allclose(got.cpu(), want, atol=1e-6)
    assert torch.equal(ids.cpu(), want_ids)
    assert torch.equal(k.moe_route(z.to(DEV), top, groups, keep).cpu(), got.cpu())
    # the plain model's router, written independently, chooses the same (but for the row of ties, which it may break otherwise)
    rows = [t for t in range(70) if t != 3]
    assert torch.equal((pg.route(z.double(), top, groups, keep) > 0)[rows], (want > 0)[rows])


def test_router_keeps_to_the_best_groups_where_a_better_expert_lies_outside():
    k = _k()
    z = torch.tensor([[0.0, 5.0, 1.0, 1.1, 4.0, 0.2, 3.0, 3.1]])
    w = k.moe_route(z.to(DEV), 3, 4, 2).cpu()
    assert torch.nonzero(w[0]).flatten().tolist() == [1, 4, 5]          # 7 and 6 score higher than 5, in a group that is out
    assert torch.allclose(w[0, [1, 4, 5]], torch.softmax(z, -1)[0, [1, 4, 5]]) and float(w.sum()) < 1


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_expert_activation_and_products_per_head(dtype):
    k = _k()
    g = torch.Generator().manual_seed(6)
    T, E, ff, shared = 13, 5, 6, 9
    F = E * ff + shared
    gu = (torch.randn(T, 2 * F, generator=g) * 2).to(dtype)
    w = plain_ops.moe_route(torch.randn(T, E, generator=g), 2)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    for sh, lim, lim_s in ((shared, 0.7, 2.5), (0, 3.0, 0.0)):
        Fx = E * ff + sh
        x = torch.cat([gu[:, :Fx], gu[:, F:F + Fx]], 1).contiguous()
        want = plain_ops.moe_expert_act(x, w, E, ff, lim, lim_s)
        got = k.moe_expert_act(x.to(DEV), w.to(DEV), E, ff, lim, lim_s)
        assert torch.allclose(got.cpu().double(), want.double(), atol=tol, rtol=tol)
        assert (got.cpu()[:, :E * ff].view(T, E, ff).abs().sum(-1) > 0).eq(w > 0).all()      # zero where not chosen
    # one expert for all, gates and ups in alternating blocks of 8
    x = gu[:, :2 * 24].contiguous()
    none = torch.empty((T, 0))
    want = plain_ops.moe_expert_act(x, none, 0, 8, 0.0, 1.3, block=8)
    got = k.moe_expert_act(x.to(DEV), none.to(DEV), 0, 8, 0.0, 1.3, block=8)
    assert torch.allclose(got.cpu().double(), want.double(), atol=tol, rtol=tol)
    g_, u_ = x.double().view(T, 3, 2, 8)[:, :, 0].reshape(T, 24), x.double().view(T, 3, 2, 8)[:, :, 1].reshape(T, 24)
    direct = torch.clamp(g_, max=1.3) * torch.sigmoid(1.702 * torch.clamp(g_, max=1.3)) * (torch.clamp(u_, -1.3, 1.3) + 1)
    assert torch.allclose(want.double(), direct, atol=tol, rtol=tol)
    H, N, K = 3, 10, 24
    x = torch.randn(T, H * K + 8, generator=g).to(dtype)
    wt = (torch.randn(H, N, K, generator=g) / K ** 0.5).to(dtype)
    for out_dtype in (torch.float32, dtype):
        want = plain_ops.head_linear(x[:, 8:], wt, torch.float64)
        got = k.head_linear(x.to(DEV)[:, 8:], wt.to(DEV), out_dtype)
        assert torch.allclose(got.cpu().double(), want, atol=tol, rtol=tol)


@pytest.mark.parametrize("E,top,ff,groups,keep,shared", [(8, 2, 24, 4, 2, 40), (6, 3, 64, 1, 1, 0), (16, 4, 8, 8, 3, 8), (3, 1, 136, 1, 1, 16),
                                                           (4, 2, 128, 1, 1, 0), (8, 2, 256, 4, 2, 40), (4, 2, 128, 2, 1, 2560)])
@pytest.mark.parametrize("T", [1, 5, 70, 333, 700])
def test_grouped_products_of_the_routed_experts(E, top, ff, groups, keep, shared, T):
    """The path of large experts on small ones: pairs sorted expert by expert on the device, tiles of pairs against
    their expert's matrices, outputs added per token; against the plain feed-forward and against the path that runs
    all experts side by side.  Experts whose width is a multiple of 128 keep their rows in blocks, and steps of 128 tokens
    and more multiply them on the tcgen05 kernel; a shared expert wide enough to fill the GPU's rounds takes that kernel too,
    with its activation in the epilogue."""
    from fastmlx_b200.engine.loading import make_runtime
    from fastmlx_b200.parts import RoutedExperts
    d = 72
    rt = make_runtime("bfloat16")
    g = torch.Generator().manual_seed(E * 100 + T)
    mlp = {"router": {"experts": E, "top": top, "groups": {"count": groups, "keep": keep}}, "expert": {"ff": ff, "limit": 0.9},
           "shared": {"ff": shared, "limit": 1.7} if shared else None}
    parts = {}
    for sparse in (True, False):
        parts[sparse] = RoutedExperts(d, E, top, ff, 0.9, "m", groups=groups, keep=keep, shared_ff=shared, shared_limit=1.7,
                                      sparse=sparse)
    W = {}
    for spec in parts[True].weight_specs():
        t = torch.randn(spec.shape, generator=g) / spec.shape[-1] ** 0.5
        W[spec.name] = (t * (12.0 if spec.name.endswith("router") else 1.5)).bfloat16()
    for p in parts.values():
        p.bind(W, rt)
    assert parts[True].sparse and not parts[False].sparse
    x = torch.randn(T, d + 8, generator=g).bfloat16()
    margins = []
    want = pg.moe_ff(x[:, :d].double(), {n[2:]: t.double() for n, t in W.items()}, mlp, margins)
    sure = margins[0] > CLOSE_CALL
    got = {s: p.forward(x.to(DEV)[:, :d], None).cpu().double() for s, p in parts.items()}
    scale = want.abs().max().item()
    assert ((got[True] - want).abs().max(1).values[sure] < 2e-2 * scale).all()
    assert ((got[True] - got[False]).abs().max(1).values[sure] < 1.5e-2 * scale).all()
    assert sure.double().mean().item() > 0.5 or T < 8


def _ctx(manager, reqs, lens, status):
    from fastmlx_b200.engine.batch import StepEntry, build_context
    entries = [StepEntry(r, [0] * n, []) for r, n in zip(reqs, lens)]
    for e in entries:
        manager.reserve(e.request, len(e.tokens))
    return build_context(entries, manager, torch.device(DEV), status)


def _attention_case(window, keep, lens_by_step, standout, hd=16, vd=24, nh=4, nkv=2, page=16, dtype=torch.float32, rot=0,
                    latent=False, gated=True, eps=1e-5, wide=False):
    """Requests fed in the given portions through the cache manager, `qk_prepare` (biases, q/k norm with a weight in
    front of an interleaved rotation) and the attention kernel; the query at position p of request 0 is aligned with
    the key at `standout(p)` so strongly that, where that key is seen, the output is its value.  `latent`: one kv
    head whose keys are the values too, written by `rmsnorm_rows` through the slot map.
    `wide`: the tiled tensor-core kernel with two-term products instead of the one-warp-per-query kernel.
    -> (outputs per request, plain outputs, the values)."""
    from fastmlx_b200 import kernels as k
    from fastmlx_b200.cache.manager import CacheManager
    from fastmlx_b200.parts.base import PagedKVSpec
    from fastmlx_b200.parts.rope import inverse_frequencies
    dev = torch.device(DEV)
    g = torch.Generator().manual_seed(window * 7 + hd + keep)
    if latent:
        nkv, vd, rot, gated, keep = 1, hd, 0, False, 0
    totals = [sum(x) for x in zip(*lens_by_step)]
    qw, kw = 1 + 0.3 * torch.randn(hd, generator=g), 1 + 0.3 * torch.randn(hd, generator=g)
    bias = 0.1 * torch.randn((nh + nkv) * hd + nkv * vd, generator=g)
    seqs = []
    for r, n in enumerate(totals):
        q = torch.randn(n, nh, hd, generator=g)
        kk = torch.randn(n, nkv, hd, generator=g)
        v = torch.randn(n, nkv, vd, generator=g)
        if r == 0 and standout is not None:
            base = kk.clone()
            for p in range(n):
                j = standout(p)
                if 0 <= j < n:
                    q[p] = base[j].repeat_interleave(nh // nkv, 0)
                    kk[j] = base[j]
        gate = torch.randn(n, nh * vd, generator=g)
        seqs.append((q, kk, v, gate))
    scale = 3.0 if standout is not None else 0.5        # normalised heads: the aligned score is about scale * hd
    want = []
    for q, kk, v, gate in seqs:
        n = q.shape[0]
        pos = torch.arange(n)
        if latent:
            kd = pg.rms_norm(kk.double(), eps, kw.double())
            qd, vv = q.double(), kd
        else:
            row = torch.cat([q.reshape(n, -1), kk.reshape(n, -1), v.reshape(n, -1)], 1).double() + bias.double()
            qd = pg.rotate_pairs(pg.rms_norm(row[:, :nh * hd].view(n, nh, hd), eps, qw.double()), pos, 10000.0, rot)
            kd = pg.rotate_pairs(pg.rms_norm(row[:, nh * hd:(nh + nkv) * hd].view(n, nkv, hd), eps, kw.double()), pos, 10000.0, rot)
            vv = row[:, (nh + nkv) * hd:].view(n, nkv, vd)
        if dtype == torch.bfloat16:
            kd, vv = kd.to(dtype).double(), vv.to(dtype).double()      # keys and values are stored in the cache's type
        seen = pg.visible(n, window or None, keep)
        o = torch.zeros(n, nh, vd, dtype=torch.float64)
        for h in range(nh):
            o[:, h] = pg.softmax_attention(qd[:, h], kd[:, h // (nh // nkv)], vv[:, h // (nh // nkv)], scale, seen)
        o = o.reshape(n, -1)
        want.append(o * torch.sigmoid(gate.double()) if gated else o)
    spec = PagedKVSpec(nkv, hd, window, 0 if vd == hd else vd, keep if window else 0, latent)
    longest = max(max(s) for s in lens_by_step)
    pages = 3 + sum(-(-(min(t, window + longest) if window else t) // page) + 2 + -(-keep // page) for t in totals)
    m = CacheManager([(spec, None, None)], page_size=page, num_pages=pages, max_requests=len(totals) + 1, dtype=dtype, device=dev)
    m.reserve(m.add_request("spare"), 3 * page)      # the first pages are not the requests' own
    reqs = [m.add_request(i) for i in range(len(totals))]
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    inv_freq = inverse_frequencies(rot, 10000.0).float().to(dev) if rot else None
    got = [[] for _ in totals]
    at = [0] * len(totals)
    kv = m.entries[0].kv
    for step_lens in lens_by_step:
        live = [(r, n) for r, n in zip(range(len(totals)), step_lens) if n > 0]
        ctx = _ctx(m, [reqs[r] for r, _ in live], [n for _, n in live], status)
        grp = ctx.groups[0]
        part = [torch.cat([seqs[r][i][at[r]:at[r] + n].reshape(n, -1) for r, n in live]) for i in range(4)]
        if latent:
            k.rmsnorm_rows(part[1].to(dev), kw.to(dev), eps, out=kv, row_map=grp.slot_mapping, status=status)
            q32 = part[0].to(dev).contiguous()
            if wide:
                assert k.wide_attention_takes(q32, kv, hd, hd)
                out = k.paged_attention_wide(q32, kv, ctx, grp, nh, 1, hd, scale, 0.0, window)
            else:
                out = k.paged_attention_general(q32, kv, ctx, grp, nh, 1, hd, hd, scale, 0.0, window, page, values_are_keys=True)
        else:
            qkv = torch.cat(part[:3], 1).to(dev).contiguous()         # 32-bit, as the product leaves it
            q32 = k.qk_prepare(qkv, ctx.positions, inv_freq, rot, True, eps, grp.slot_mapping, kv, nh, nkv, hd, vd, status,
                               bias=bias.to(dev), q_weight=qw.to(dev), k_weight=kw.to(dev), norm_first=True)
            gate = part[3].to(dev).contiguous() if gated else None
            if wide:
                joined = torch.zeros((q32.shape[0], nh * vd + 6), dtype=dtype, device=dev)
                assert k.wide_attention_takes(q32, kv, hd, vd, joined[:, 2:2 + nh * vd])
                out = k.paged_attention_wide(q32, kv, ctx, grp, nh, nkv, hd, scale, 0.0, window, out=joined[:, 2:2 + nh * vd],
                                             keep_first=spec.keep_first, gate=gate)
                assert joined[:, :2].abs().max().item() == 0 and joined[:, 2 + nh * vd:].abs().max().item() == 0
            else:
                out = k.paged_attention_general(q32, kv, ctx, grp, nh, nkv, hd, vd, scale, 0.0, window, page,
                                                keep_first=spec.keep_first, gate=gate)
        out = out.cpu().double()
        off = 0
        for r, n in live:
            got[r].append(out[off:off + n])
            off += n
            at[r] += n
            m.commit(reqs[r])
        m.check()
    assert status.tolist()[0] == 0
    return [torch.cat(x) for x in got], want, seqs


KERNELS = [(torch.float32, False), (torch.bfloat16, False), (torch.bfloat16, True)]
KERNEL_IDS = ["float32", "bfloat16", "bfloat16-tiled"]
HOW = {"prompt": [[150, 40]], "portions": [[31, 3], [2, 1], [37, 30], [38, 2], [42, 4]], "decoded": [[60, 1]] + [[1, 0]] * 90}


@pytest.mark.parametrize("dtype,wide", KERNELS, ids=KERNEL_IDS)
@pytest.mark.parametrize("edge", ["inside", "outside"])
@pytest.mark.parametrize("how", ["prompt", "portions", "decoded"])
@pytest.mark.parametrize("latent", [False, True])
def test_attention_window_edge(dtype, wide, edge, how, latent):
    """The key that stands out sits on the last place the window still holds, or one before it: its value must be the
    output, or must not be in it.  Pages that the window has passed are given back on the way."""
    window = 37
    standout = (lambda p: p - window + 1) if edge == "inside" else (lambda p: p - window)
    kw = dict(dtype=dtype, rot=8, latent=latent, gated=False, wide=wide, hd=64, vd=64 if wide else 24)
    got, want, _ = _attention_case(window, 3, HOW[how], standout, **kw)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    for r in range(2):
        n_r = got[r].shape[0]
        assert torch.allclose(got[r], want[r][:n_r], atol=tol, rtol=tol), r
    # the oracle itself shows the edge: the outputs of the two cases differ where the key is seen
    other, _, _ = _attention_case(window, 3, HOW[how], (lambda p: p - window) if edge == "inside" else (lambda p: p - window + 1), **kw)
    assert (got[0][100] - other[0][100]).abs().max().item() > 0.1


@pytest.mark.parametrize("dtype,wide", KERNELS, ids=KERNEL_IDS)
@pytest.mark.parametrize("edge", ["inside", "outside"])
@pytest.mark.parametrize("how", ["prompt", "portions", "decoded"])
@pytest.mark.parametrize("keep,page", [(3, 16), (19, 16), (1, 8), (16, 16), (70, 16)])
def test_attention_kept_first_tokens(dtype, wide, edge, how, keep, page):
    """The key that stands out is the last kept token, or the first that is not kept (seen only while the window
    still holds it): kept tokens are seen from far away, at their true positions, through pages that are never given
    back; the token after them is not."""
    window = 37
    j = keep - 1 if edge == "inside" else keep
    got, want, seqs = _attention_case(window, keep, HOW[how], lambda p: j, dtype=dtype, rot=4, page=page, wide=wide, hd=64,
                                      vd=64 if wide else 24)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    for r in range(2):
        n_r = got[r].shape[0]
        assert torch.allclose(got[r], want[r][:n_r], atol=tol, rtol=tol), r
    # the oracle itself shows the edge: far behind the window, the output is the kept key's value, or nothing of the
    # next token's
    value = want[0][j] / torch.sigmoid(seqs[0][3][j].double())          # position j attends to itself alone, nearly
    far = want[0][120] / torch.sigmoid(seqs[0][3][120].double())
    assert ((far - value).abs().max().item() < 0.1) == (edge == "inside")


@pytest.mark.parametrize("dtype,wide", KERNELS, ids=KERNEL_IDS)
@pytest.mark.parametrize("latent", [False, True])
def test_attention_far_key_among_hundreds(dtype, wide, latent):
    """No window: every query's key that stands out is position 1 (far back for late queries, among the first tokens
    for early ones); three requests of unequal length, page borders, values narrower than keys."""
    got, want, _ = _attention_case(0, 0, [[330, 5, 64], [1, 1, 64], [2, 0, 1], [64, 16, 0]], lambda p: 1, hd=32, vd=32 if wide else 8, nh=2,
                                   nkv=1, dtype=dtype, rot=32, latent=latent, wide=wide)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    for r in range(3):
        assert torch.allclose(got[r], want[r], atol=tol, rtol=tol), r


@pytest.mark.parametrize("hd", [40, 300, 512])
def test_attention_over_wide_latents(hd):
    got, want, _ = _attention_case(21, 0, [[50, 9], [1, 1], [7, 0]], None, hd=hd, nh=3, latent=True)
    for r in range(2):        # scores of hundreds of terms, and peaked weights: the 32-bit sums' rounding shows at 1e-4
        assert torch.allclose(got[r], want[r], atol=3e-4, rtol=3e-4), r


# ----------------------------------------------------------------------------- the engine
def _plain_greedy(cfg, W, prompt, n):
    toks, out, margins = list(prompt), [], []
    for _ in range(n):
        row = pg.forward(cfg, W, toks)[-1]
        top = torch.topk(row, 2).values
        margins.append(float(top[0] - top[1]) / float(row.abs().max()))
        out.append(int(torch.argmax(row)))
        toks.append(out[-1])
    return out, margins


@pytest.mark.parametrize("dtype,slack", [("float32", 1e-5), ("bfloat16", 4e-2)])
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_engine(models, dtype, slack, graphs):
    """Six prompts over three slots, portions of 16 tokens: the scheduler admits, cuts and batches; slots and pages
    are used again; decode steps replay CUDA graphs where asked."""
    from fastmlx_b200 import Engine, SamplingParams
    d, W, _, _ = models["G1"]
    cfg = tg.G1
    prompts = [tiny.rand_tokens(n, cfg["vocab"], 500 + n) for n in (1, 9, 40, 23, 3, 57)]
    eng = Engine(d, dtype=dtype, block_size=16, max_cache_tokens=512, max_concurrent_requests=3, prefill_chunk=16,
                 cuda_graphs=graphs)
    outs = eng.generate(prompts, SamplingParams(max_tokens=12, temperature=0.0))
    for p, out in zip(prompts, outs):
        assert out.finished and out.completion_tokens == 12
        want, margins = _plain_greedy(cfg, W, p, 12)
        for i, (a, b) in enumerate(zip(out.output_token_ids, want)):
            if a != b:
                assert margins[i] < slack, (i, a, b, margins[i])
                break                                   # after a tie that went the other way the texts differ
    st = eng.stats()
    assert st["pages_used"] == 0
    if graphs:
        assert st["graph_replays"] > 0


def test_command_line_and_trace_program(models, tmp_path):
    """`python -m fastmlx_b200 generate` and bin/trace_run on a Gekavik folder, as a user runs them."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    d, W, prompts, ref = models["G4"]
    out = subprocess.run([sys.executable, "-m", "fastmlx_b200", "generate", "--model-dir", d, "--dtype", "float32", "--prompt-ids",
                          "5,6,7;9", "--max-tokens", "5", "--temperature", "0", "--max-cache-tokens", "256"], cwd=root,
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [json.loads(x) for x in out.stdout.splitlines() if x.startswith("{")]
    assert [len(x["output_token_ids"]) for x in lines] == [5, 5]
    want, margins = _plain_greedy(tg.G4, W, [5, 6, 7], 5)
    for i, (a, b) in enumerate(zip(lines[0]["output_token_ids"], want)):
        if a != b:
            assert margins[i] < 1e-5
            break
    sub = {r: prompts[r] for r in ("r1", "r2", "r3")}
    steps = traces.mixed(sub)
    outdir = tmp_path / "out"
    proc = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", d, "--dtype", "float32", "--out", str(outdir),
                           "--max-tokens", "256"], input="".join(json.dumps(s) + "\n" for s in steps), cwd=root,
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [x for x in proc.stdout.splitlines() if x.startswith("done ")] == [f"done {s['step']}" for s in steps]
    outs = [np.fromfile(outdir / f"{s['step']}.f32", dtype="<f4").reshape(-1, tg.G4["vocab"]) for s in steps]
    _compare(steps, outs, sub, ref, TOL["float32"])

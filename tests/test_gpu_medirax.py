"""Medirax on the GPU against the plain model of tests/plain_medirax.py: each mechanism's kernels
alone, whole prompts against decoding token by token, portions down to two tokens, mixed batches
over pools and slots that are used again, window edges and far keys made to stand out, long
decoding, and greedy generation through the engine."""
import math

import numpy as np
import pytest
import torch

import plain_medirax as pm
import tiny
import tiny_medirax as tm
import traces

pytestmark = pytest.mark.gpu

# Largest |difference| as a fraction of the largest |logit| of the plain model (float64).  32-bit: float32
# sums against float64.  bfloat16: weights are bfloat16 in both; the engine rounds activations.
TOL = {"float32": 2e-5, "bfloat16": 4e-2}
CASES = {
    "M1": dict(lens=[1, 2, 7, 45, 38, 100, 39, 76, 131], page=16, max_tokens=448),
    "M2": dict(lens=[3, 17, 72, 140, 71, 33, 90], page=16, max_tokens=384),
    "M3": dict(lens=[5, 64, 33, 97, 20, 50, 70], page=32, max_tokens=384),
    "M4": dict(lens=[4, 40, 23, 66, 35, 80], page=16, max_tokens=256),
}


def _prompts(name):
    return {f"r{i}": tiny.rand_tokens(n, tm.CONFIGS[name]["vocab"], 300 + i) for i, n in enumerate(CASES[name]["lens"])}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("medirax")
    out = {}
    for name, cfg in tm.CONFIGS.items():
        d = tiny.make_model_dir(root, cfg, seed=23)
        W = tiny.load_plain_weights(d)
        prompts = _prompts(name)
        out[name] = (d, W, prompts, {r: pm.forward(cfg, W, t) for r, t in prompts.items()})
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


def _compare(steps, outs, prompts, ref, tol):
    rows = traces.collect(steps, outs)
    for rid, toks in prompts.items():
        assert sorted(rows[rid]) == list(range(len(toks)))
        got = torch.from_numpy(np.stack([rows[rid][i] for i in range(len(toks))])).double()
        err = (got - ref[rid]).abs().max(dim=1).values / ref[rid].abs().max().item()
        bad = torch.nonzero(err > tol)
        assert bad.numel() == 0, (f"request {rid}: first wrong position {int(bad[0])} of {len(toks)}, "
                                  f"error {err[int(bad[0])].item():.3e} (allowed {tol:.1e})")


CUTS = {"whole": traces.whole, "tail": traces.tail_decoded, "portions": traces.portions, "mixed": traces.mixed,
        "ones": lambda p: traces.tail_decoded(p, tail=10 ** 6)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["M1", "M2", "M3", "M4"])
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed", "ones"])
def test_replay(models, name, dtype, cut):
    d, W, prompts, ref = models[name]
    case = CASES[name]
    steps = CUTS[cut](prompts)
    outs, rp = _run(d, dtype, steps, case["max_tokens"], case["page"])
    _compare(steps, outs, prompts, ref, TOL[dtype])
    if cut == "mixed":
        need = sum(-(-len(t) // case["page"]) for t in prompts.values())
        assert all(need > g.pool.num_pages for g in rp.manager.groups), "the pool is too large for pages to be used again"
        assert len(prompts) > rp.manager.max_requests, "too many slots for one to be used again"


@pytest.mark.parametrize("name", ["M1", "M2"])
def test_cuts_agree_in_32_bit_to_the_bit(models, name):
    """No sum's order depends on the cut, the batch, the pages or the slot: in 32-bit the logits are equal."""
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


def test_long_decoding_carries_state_and_window(models):
    """150 tokens decoded one by one behind a short prompt: the window of 70 passes over decoded tokens, the
    delta rule's state is carried through every step."""
    d, W, prompts, ref = models["M2"]
    sub = {"r3": prompts["r3"]}
    steps = traces.tail_decoded(sub, tail=130)
    outs, _ = _run(d, "float32", steps, 256, 16)
    _compare(steps, outs, sub, ref, TOL["float32"])


# ----------------------------------------------------------------------------- mechanisms alone
def _ctx(manager, reqs, lens, device, status):
    from fastmlx_b200.engine.batch import StepEntry, build_context
    entries = [StepEntry(r, [0] * n, []) for r, n in zip(reqs, lens)]
    for e in entries:
        manager.reserve(e.request, len(e.tokens))
    return build_context(entries, manager, device, status)


@pytest.mark.parametrize("H,G,D,Dv", [(2, 1, 24, 40), (3, 3, 128, 16), (1, 1, 200, 9), (4, 2, 8, 64)])
def test_delta_rule_kernel(H, G, D, Dv):
    """The recurrence alone: three requests of unequal length in two steps, from and into state slots."""
    from fastmlx_b200 import kernels as k
    from fastmlx_b200.cache.manager import CacheManager
    from fastmlx_b200.parts.base import StateSpec
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(H * 1000 + D)
    C = 2 * G * D + H * Dv
    lens = [[5, 1, 33], [2, 17, 1]]
    total = [sum(x) for x in zip(*lens)]
    seqs = []
    for n in total:
        q = pm.unit_vector(torch.randn(n, G, D, generator=g, dtype=torch.float64)) * D ** -0.5
        kk = pm.unit_vector(torch.randn(n, G, D, generator=g, dtype=torch.float64))
        v = torch.randn(n, H, Dv, generator=g, dtype=torch.float64)
        decay = torch.rand(n, H, generator=g, dtype=torch.float64) * 0.5 + 0.5
        beta = torch.rand(n, H, generator=g, dtype=torch.float64)
        seqs.append((q, kk, v, decay, beta))
    want = []
    for q, kk, v, decay, beta in seqs:
        o = torch.zeros(q.shape[0], H, Dv, dtype=torch.float64)
        for h in range(H):
            S = torch.zeros(D, Dv, dtype=torch.float64)
            for t in range(q.shape[0]):
                S = decay[t, h] * S
                S = S + torch.outer(kk[t, h // (H // G)], beta[t, h] * (v[t, h] - S.T @ kk[t, h // (H // G)]))
                o[t, h] = S.T @ q[t, h // (H // G)]
        want.append(o)
    m = CacheManager([(None, StateSpec((H * Dv * D + 7,)), None)], page_size=16, num_pages=1, max_requests=4, device=dev)
    m.add_request("spare")                      # the requests do not sit in slots 0, 1, 2
    reqs = [m.add_request(i) for i in range(3)]
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    at = [0, 0, 0]
    for step_lens in lens:
        ctx = _ctx(m, reqs, step_lens, dev, status)
        qkv = torch.cat([torch.cat([s[0][a:a + n].reshape(n, -1), s[1][a:a + n].reshape(n, -1), s[2][a:a + n].reshape(n, -1)], 1)
                         for s, a, n in zip(seqs, at, step_lens)]).float().to(dev).contiguous()
        gb = torch.cat([torch.cat([s[3][a:a + n], s[4][a:a + n]], 1) for s, a, n in zip(seqs, at, step_lens)]).float().to(dev)
        assert qkv.shape[1] == C
        o = k.delta_rule(qkv, gb.contiguous(), ctx, m.entries[0].state, H, G, D, Dv).cpu().double()
        off = 0
        for i, n in enumerate(step_lens):
            ref = want[i][at[i]:at[i] + n].reshape(n, -1)
            assert torch.allclose(o[off:off + n], ref, atol=2e-5 * ref.abs().max().item()), (i, at[i])
            off += n
            at[i] += n
        for r in reqs:
            m.commit(r)
    assert status.tolist()[0] == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps", [1, 2, 4])
def test_delta_prepare_kernel(dtype, taps):
    """Convolution through the state slot (portions of 1, 2 and more tokens), SiLU, unit vectors, decay and beta."""
    from fastmlx_b200 import kernels as k
    from fastmlx_b200.cache.manager import CacheManager
    from fastmlx_b200.parts.base import StateSpec
    dev = torch.device("cuda")
    H, G, D, Dv = 3, 1, 20, 12
    C = 2 * G * D + H * Dv
    g = torch.Generator().manual_seed(taps)
    n = 23
    proj = (torch.randn(n, C + 5, generator=g) * 2).to(dtype)
    ab = torch.randn(n, 2 * H, generator=g) * 3
    conv_w = torch.randn(C, taps, generator=g)
    a_log, dt_bias = torch.randn(H, generator=g), torch.randn(H, generator=g)
    x = pm.causal_conv_silu(proj[:, :C].double(), conv_w.double())
    q = pm.unit_vector(x[:, :G * D].view(n, G, D)) * D ** -0.5
    kk = pm.unit_vector(x[:, G * D:2 * G * D].view(n, G, D))
    want = torch.cat([q.reshape(n, -1), kk.reshape(n, -1), x[:, 2 * G * D:]], 1)
    want_gb = torch.cat([torch.exp(-torch.exp(a_log.double()) * torch.nn.functional.softplus(ab[:, H:].double() + dt_bias.double())),
                         torch.sigmoid(ab[:, :H].double())], 1)
    s_floats = 11
    m = CacheManager([(None, StateSpec((s_floats + (taps - 1) * C,)), None)], page_size=16, num_pages=1, max_requests=3, device=dev)
    other = m.add_request("other")
    req = m.add_request("x")
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    at = 0
    for cut in (1, 2, 1, 5, 2, 12):
        ctx = _ctx(m, [req], [cut], dev, status)
        qkv, gb = k.delta_prepare(proj[at:at + cut].to(dev), ab[at:at + cut].to(dev).contiguous(), conv_w.to(dev), a_log.to(dev),
                                  dt_bias.to(dev), ctx, m.entries[0].state, s_floats, H, G, D, Dv, taps)
        assert torch.allclose(qkv.cpu().double(), want[at:at + cut], atol=1e-5), at
        assert torch.allclose(gb.cpu().double(), want_gb[at:at + cut], atol=1e-6), at
        m.commit(req)
        at += cut
    assert at == n and status.tolist()[0] == 0
    assert m.entries[0].state[other.slot].abs().max().item() == 0          # another request's slot is not touched


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_norm_and_activations(dtype):
    from fastmlx_b200 import kernels as k
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(5)
    T, H, Dv = 7, 3, 40
    o = torch.randn(T, H * Dv, generator=g) * 3
    gate = torch.randn(T, H * Dv + 8, generator=g).to(dtype)
    w = torch.randn(Dv, generator=g)
    want = pm.rms_norm(o.double().view(T, H, Dv), 1e-3, w.double()) * pm.silu(gate[:, 8:].double().view(T, H, Dv))
    wide = torch.zeros(T, H * Dv + 16, dtype=dtype, device=dev)
    got = k.gated_rmsnorm(o.to(dev), gate.to(dev)[:, 8:], w.to(dev), 1e-3, H, Dv, dtype, out=wide[:, 16:])
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert torch.allclose(got.cpu().double().view(T, H, Dv), want, rtol=tol, atol=tol)
    assert wide[:, :16].abs().max().item() == 0
    x = (torch.randn(9, 50, generator=g) * 3).to(dtype)
    for kind, fn in (("relu2", pm.relu_squared), ("silu", pm.silu),
                     ("gelu_tanh", lambda z: 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3))))):
        got = k.activation(x.to(dev)[:, 3:44], kind).cpu().double()
        assert torch.allclose(got, fn(x[:, 3:44].double()), rtol=tol, atol=tol), kind


def _attention_case(window, cap, lens_by_step, standout, hd=16, vd=24, nh=4, nkv=2, page=16, dtype=torch.float32,
                    rot=0, norm_eps=None, wide=False):
    """Requests fed in the given portions through the cache manager and the two attention kernels; the query at
    position p of request 0 is aligned with the key at `standout(p)` so strongly that, where that key is seen, the
    output is its value.  -> (outputs per request [n, nh*vd], plain outputs)."""
    from fastmlx_b200 import kernels as k
    from fastmlx_b200.cache.manager import CacheManager
    from fastmlx_b200.parts.base import PagedKVSpec
    from fastmlx_b200.parts.rope import inverse_frequencies
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(window * 7 + hd)
    totals = [sum(x) for x in zip(*lens_by_step)]
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
                    q[p] = 6.0 * base[j].repeat_interleave(nh // nkv, 0) / base[j].repeat_interleave(nh // nkv, 0).norm(dim=-1, keepdim=True)
                    kk[j] = base[j] * 3.0
        seqs.append((q.to(dtype), kk.to(dtype), v.to(dtype)))
    scale = 0.5
    want = []
    for q, kk, v in seqs:
        n = q.shape[0]
        pos = torch.arange(n)
        qd, kd = q.double(), kk.double()
        if rot:
            qd, kd = pm.rotate_half_partial(qd, pos, 10000.0, rot), pm.rotate_half_partial(kd, pos, 10000.0, rot)
        if norm_eps is not None:
            qd, kd = pm.rms_norm(qd, norm_eps), pm.rms_norm(kd, norm_eps)
        if dtype == torch.bfloat16:
            kd = kd.to(dtype).double()             # keys are stored in the cache's type
        o = torch.zeros(n, nh, vd, dtype=torch.float64)
        for h in range(nh):
            s = qd[:, h] @ kd[:, h // (nh // nkv)].T * scale
            if cap:
                s = cap * torch.tanh(s / cap)
            d = pos[:, None] - pos[None, :]
            seen = (d >= 0) & ((d < window) if window else True)
            o[:, h] = torch.softmax(s.masked_fill(~seen, -math.inf), -1) @ v[:, h // (nh // nkv)].double()
        want.append(o.reshape(n, -1))
    spec = PagedKVSpec(nkv, hd, window, 0 if vd == hd else vd)
    pages = 3 + sum(-(-(min(t, window + max(max(s) for s in lens_by_step)) if window else t) // page) + 1 for t in totals)
    m = CacheManager([(spec, None, None)], page_size=page, num_pages=pages, max_requests=len(totals) + 1, dtype=dtype, device=dev)
    m.reserve(m.add_request("spare"), 3 * page)      # the first pages are not the requests' own
    reqs = [m.add_request(i) for i in range(len(totals))]
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    inv_freq = inverse_frequencies(rot, 10000.0).float().to(dev) if rot else None
    got = [[] for _ in totals]
    at = [0] * len(totals)
    for step_lens in lens_by_step:
        live = [(r, n) for r, n in zip(range(len(totals)), step_lens) if n > 0]
        ctx = _ctx(m, [reqs[r] for r, _ in live], [n for _, n in live], dev, status)
        qkv = torch.cat([torch.cat([seqs[r][0][at[r]:at[r] + n].reshape(n, -1), seqs[r][1][at[r]:at[r] + n].reshape(n, -1),
                                    seqs[r][2][at[r]:at[r] + n].reshape(n, -1)], 1) for r, n in live]).to(dev).contiguous()
        grp = ctx.groups[0]
        q32 = k.qk_prepare(qkv, ctx.positions, inv_freq, rot, False, norm_eps, grp.slot_mapping, m.entries[0].kv, nh, nkv, hd, vd, status)
        if wide:                                     # the tiled tensor-core kernel with two-term products
            assert k.wide_attention_ok(q32, m.entries[0].kv, hd, vd)
            joined = torch.zeros((q32.shape[0], nh * vd + 6), dtype=dtype, device=dev)
            out = k.paged_attention_wide(q32, m.entries[0].kv, ctx, grp, nh, nkv, hd, scale, cap, window, out=joined[:, 2:2 + nh * vd])
            assert joined[:, :2].abs().max().item() == 0 and joined[:, 2 + nh * vd:].abs().max().item() == 0
            out = out.cpu().double()
        else:
            out = k.paged_attention_general(q32, m.entries[0].kv, ctx, grp, nh, nkv, hd, vd, scale, cap, window, page).cpu().double()
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


@pytest.mark.parametrize("dtype,wide", KERNELS, ids=KERNEL_IDS)
@pytest.mark.parametrize("edge", ["inside", "outside"])
@pytest.mark.parametrize("how", ["prompt", "portions", "decoded"])
def test_attention_window_edge(dtype, wide, edge, how):
    """The key that stands out sits on the last place the window still holds, or one before it: its value must be
    the output, or must not be in it.  Pages that the window has passed are given back on the way."""
    window, n = 37, 150
    standout = (lambda p: p - window + 1) if edge == "inside" else (lambda p: p - window)
    steps = {"prompt": [[n, 40]], "portions": [[31, 3], [2, 1], [37, 30], [38, 2], [42, 4]],
             "decoded": [[60, 1]] + [[1, 0]] * 90}[how]
    vd = 16 if wide else 24
    got, want, seqs = _attention_case(window, 40.0, steps, standout, dtype=dtype, vd=vd, wide=wide)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    for r in range(2):
        n_r = got[r].shape[0]
        assert torch.allclose(got[r], want[r][:n_r], atol=tol, rtol=tol), r
    # the oracle itself shows the edge: where the key is seen the output is its value
    v = seqs[0][2].double()
    p = 100
    close = (want[0][p].view(4, vd)[0] - v[standout(p), 0]).abs().max().item()
    assert (close < 1e-2) == (edge == "inside")


@pytest.mark.parametrize("dtype,wide", KERNELS, ids=KERNEL_IDS)
def test_attention_far_key_among_hundreds_and_first_tokens(dtype, wide):
    """No window: every query's standing-out key is position 1 (far back for late queries, the first tokens for
    early ones); values narrower than keys (as wide on the tiled kernel), capped scores, three requests of unequal
    length, page borders."""
    got, want, _ = _attention_case(0, 25.0, [[330, 5, 64], [1, 1, 64], [2, 0, 1], [64, 16, 0]], lambda p: 1, hd=32,
                                   vd=32 if wide else 8, nh=2, nkv=1, dtype=dtype, wide=wide)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    for r in range(3):
        assert torch.allclose(got[r], want[r], atol=tol, rtol=tol), r


def test_tiled_attention_keeps_16_bits_of_queries_and_weights():
    """Against the same attention with 32-bit queries and weights over the same bfloat16 keys and values: the
    two-term products leave an error far below one bfloat16 step of the output."""
    got, want, _ = _attention_case(90, 15.0, [[200, 33], [1, 1], [40, 0]], None, hd=64, vd=64, nh=4, nkv=1, dtype=torch.bfloat16,
                                   wide=True, norm_eps=1e-6, rot=32)
    ref, _, _ = _attention_case(90, 15.0, [[200, 33], [1, 1], [40, 0]], None, hd=64, vd=64, nh=4, nkv=1, dtype=torch.bfloat16,
                                wide=False, norm_eps=1e-6, rot=32)
    for r in range(2):
        # both outputs are rounded to bfloat16 (2^-9 relative); they differ by at most one such step, and rarely
        diff = (got[r] - ref[r]).abs()
        assert (diff <= 2.0 ** -7 * ref[r].abs() + 1e-3).all(), (diff.max().item(), (diff / (ref[r].abs() + 1e-3)).max().item())
        assert (diff > 0).double().mean().item() < 0.25


def test_tiled_attention_shares_a_rows_keys_out_over_blocks():
    """Steps of single tokens behind long contexts (and such rows at the head of a mixed step): several blocks take
    shares of a row's keys and a second kernel puts their parts together."""
    from fastmlx_b200 import kernels as k
    assert k.wide_attention_splits(3, 2, 701) > 1
    steps = [[700, 300, 5]] + [[1, 1, 1]] * 6 + [[1, 1, 40]] * 2 + [[1, 0, 1]]
    got, want, _ = _attention_case(0, 20.0, steps, lambda p: 3, hd=32, vd=32, nh=4, nkv=2, dtype=torch.bfloat16, wide=True)
    for r in range(3):
        assert torch.allclose(got[r], want[r], atol=2e-2, rtol=2e-2), r
    got, want, _ = _attention_case(300, 0.0, [[650, 420]] + [[1, 1]] * 5, None, hd=64, vd=64, nh=8, nkv=1, dtype=torch.bfloat16, wide=True)
    for r in range(2):
        assert torch.allclose(got[r], want[r], atol=2e-2, rtol=2e-2), r


@pytest.mark.parametrize("kind", ["relu2", "gelu_tanh", "silu"])
def test_activation_in_the_products_epilogue(kind):
    """The decode product (at most 16 rows) and the tensor-memory product of prompt portions apply the feed-forward's
    activation themselves, into a slice of a wider buffer."""
    from fastmlx_b200 import kernels as k
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(3)
    fn = {"relu2": pm.relu_squared, "silu": pm.silu,
          "gelu_tanh": lambda z: 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))}[kind]
    x = torch.randn(5, 256, generator=g).bfloat16().to(dev)
    w = (torch.randn(300, 256, generator=g) * 0.2).bfloat16().to(dev)
    b = torch.randn(300, generator=g).to(dev)
    wide = torch.zeros(5, 320, dtype=torch.bfloat16, device=dev)
    got = k.gemv(x, w, b, act=kind, out=wide[:, 8:308])
    want = fn((x.double() @ w.double().T + b.double()).bfloat16().double())
    assert torch.allclose(got.double(), want, rtol=1e-2, atol=1e-2) and wide[:, 308:].abs().max().item() == 0
    if kind == "relu2":
        x = torch.randn(256, 512, generator=g).bfloat16().to(dev)
        w = (torch.randn(1024, 512, generator=g) * 0.1).bfloat16().to(dev)
        wide = torch.zeros(256, 1024 + 64, dtype=torch.bfloat16, device=dev)
        got = k.gemm_tcgen05(x, w, epilogue=k.EPI_RELU2, out=wide[:, 64:])
        want = fn((x.double() @ w.double().T).bfloat16().double())
        # one bfloat16 step of the product is two of its square
        assert torch.allclose(got.double(), want, rtol=3e-2, atol=3e-2) and wide[:, :64].abs().max().item() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rot,hd", [(8, 24), (16, 16), (0, 40)])
def test_rotation_and_norm_of_q_and_k(dtype, rot, hd):
    """Partial rotation in the half-split pairing, then q and k divided by their root mean square: through the
    attention kernels at positions up to 200, against the plain rotation and norm."""
    got, want, _ = _attention_case(50, 0.0, [[120, 7], [81, 30]], None, hd=hd, vd=hd, dtype=dtype, rot=rot, norm_eps=1e-5)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    for r in range(2):
        assert torch.allclose(got[r], want[r], atol=tol, rtol=tol), r


# ----------------------------------------------------------------------------- the engine
def _plain_greedy(cfg, W, prompt, n):
    toks, out, margins = list(prompt), [], []
    for _ in range(n):
        row = pm.forward(cfg, W, toks)[-1]
        top = torch.topk(row, 2).values
        margins.append(float(top[0] - top[1]) / float(row.abs().max()))
        out.append(int(torch.argmax(row)))
        toks.append(out[-1])
    return out, margins


@pytest.mark.parametrize("dtype,slack", [("float32", 1e-5), ("bfloat16", 4e-2)])
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_engine(models, dtype, slack, graphs):
    """Six prompts over three slots, portions of 16 tokens: the scheduler admits, cuts and batches; slots and
    pages are used again; decode steps replay CUDA graphs where asked."""
    from fastmlx_b200 import Engine, SamplingParams
    d, W, _, _ = models["M1"]
    cfg = tm.M1
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
    """`python -m fastmlx_b200 generate` and bin/trace_run on a Medirax folder, as a user runs them."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    d, W, prompts, ref = models["M4"]
    out = subprocess.run([sys.executable, "-m", "fastmlx_b200", "generate", "--model-dir", d, "--dtype", "float32", "--prompt-ids",
                          "5,6,7;9", "--max-tokens", "5", "--temperature", "0", "--max-cache-tokens", "256"], cwd=root,
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [json.loads(x) for x in out.stdout.splitlines() if x.startswith("{")]
    assert [len(x["output_token_ids"]) for x in lines] == [5, 5]
    want, margins = _plain_greedy(tm.M4, W, [5, 6, 7], 5)
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
    outs = [np.fromfile(outdir / f"{s['step']}.f32", dtype="<f4").reshape(-1, tm.M4["vocab"]) for s in steps]
    _compare(steps, outs, sub, ref, TOL["float32"])


def test_preemption_recomputes_state_and_changes_no_token(models):
    """A pool too small for three requests to grow together: the scheduler preempts the newest, frees its pages and its
    state slot, and recomputes it later from zero state; in 32-bit every request still produces what it produces with
    room to spare."""
    from fastmlx_b200 import Engine, SamplingParams
    d, W, _, _ = models["M2"]                        # one of its attention layers keeps every key
    prompts = [tiny.rand_tokens(n, tm.M2["vocab"], 900 + n) for n in (30, 28, 25)]
    sp = SamplingParams(max_tokens=40, temperature=0.0)
    tight = Engine(d, dtype="float32", block_size=8, initial_cache_blocks=18, max_concurrent_requests=4)
    outs = tight.generate(prompts, sp)
    assert tight.stats()["preemptions"] > 0
    roomy = Engine(d, dtype="float32", block_size=8, initial_cache_blocks=64, max_concurrent_requests=4)
    assert [o.output_token_ids for o in outs] == [o.output_token_ids for o in roomy.generate(prompts, sp)]
    assert all(o.finish_reason == "length" and len(o.output_token_ids) == 40 for o in outs)
    assert tight.stats()["pages_used"] == 0
    tight.manager.check()

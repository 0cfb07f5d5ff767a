"""Sampling kernels against plain fp32 PyTorch / the host reference implementation: arg-max ties, top-k order, top-p
cut, draws, penalties, NLL, the speculative accept rule, and the vocabulary-sharded merge."""
import random

import pytest
import torch

pytestmark = pytest.mark.gpu


def _logits(n, v, seed, ties=True):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(n, v, generator=g, device="cuda") * 3
    if ties:
        x = (x * 4).round() / 4            # many exact ties: the lowest index must win
    return x


def test_argmax_ties_and_offset():
    from velogb10_b200.ops import kernels as K
    x = _logits(5, 70001, 1)
    x[2, 123] = x[2, 60000] = 99.0
    out = torch.zeros(5, dtype=torch.int32, device="cuda")
    val = torch.zeros(5, device="cuda")
    K.argmax(x, 5, out, val, idx_offset=1000)
    for r in range(5):
        m = x[r].max()
        want = int(torch.nonzero(x[r] == m)[0])
        assert int(out[r]) == want + 1000 and float(val[r]) == float(m)
    assert int(out[2]) == 123 + 1000


@pytest.mark.parametrize("v", [1000, 50000, 248320])
def test_topk_nucleus_and_draw_match_host(v):
    from velogb10_b200.engine import sampling as S
    from velogb10_b200.engine.device_sampler import DeviceSampler
    x = _logits(6, v, v)
    params = [S.SamplingParams(0.7, 0.8, 20), S.SamplingParams(1.3, 0.5, 64), S.SamplingParams(0.0, 0.8, 20),
              S.SamplingParams(0.9, 1.0, 100), S.SamplingParams(0.5, 0.95, 1), S.SamplingParams(2.0, 0.3, 7)]
    ds = DeviceSampler("cuda", v, cap=16)
    rnd = random.Random(3)
    for trial in range(4):
        u = [rnd.random() for _ in params]
        ds.upload(params, u=u)
        tok = ds.select(x.clone(), 6, False, want_nucleus=True).tolist()
        ids, probs, keep = ds.ids.cpu(), ds.probs.cpu(), ds.keep.cpu().tolist()
        for r, p in enumerate(params):
            ref = S.nucleus_host(x[r].cpu(), p)
            assert ids[r, :keep[r]].tolist() == ref.ids, (r, keep[r], len(ref.ids))
            assert torch.allclose(probs[r, :keep[r]], torch.tensor(ref.probs), rtol=2e-5, atol=1e-7)
            dev_nuc = S.Nucleus(ids[r, :keep[r]].tolist(), probs[r, :keep[r]].tolist())
            u24 = float(torch.tensor(u[r], dtype=torch.float32))
            assert tok[r] == dev_nuc.draw(u24), (r, tok[r])
    # pick(): the host rule end to end (same keyed uniform, penalties off)
    keys = [11 * (i + 1) for i in range(6)]
    got = ds.pick(x.clone(), params, [[] for _ in params], keys)
    agree = sum(got[r] == S.nucleus_host(x[r].cpu(), p).draw(S.rng_uniform(keys[r], S.DOMAIN_SAMPLE, 0))
                for r, p in enumerate(params))
    assert agree >= 5            # a last-bit difference in a probability may move one draw across a boundary
    assert got[2] == int(torch.nonzero(x[2] == x[2].max())[0])


def test_sharded_merge_equals_unsharded():
    """Four vocabulary shards reduced separately and merged give exactly the single-GPU nucleus and token."""
    from velogb10_b200.engine import sampling as S
    from velogb10_b200.engine.device_sampler import DeviceSampler, MAXK
    from velogb10_b200.ops import kernels as K
    W, vl, n = 4, 12345, 5
    x = _logits(n, W * vl, 9)
    params = [S.SamplingParams(0.8, 0.9, 40)] * n
    u = [0.1, 0.5, 0.9, 0.33, 0.77]
    full = DeviceSampler("cuda", W * vl, cap=16)
    full.upload(params, u=u)
    t_full = full.select(x.clone(), n, False, want_nucleus=True).clone()
    sh = DeviceSampler("cuda", vl, cap=16)
    sh.upload(params, u=u)
    lists = torch.zeros(n, W, MAXK * 2, device="cuda")
    for q in range(W):
        K.topk_local(x[:, q * vl:(q + 1) * vl].contiguous(), n, sh.temp, sh.top_k, q * vl, sh.cand_chunks, sh.cand)
        lists[:, q] = sh.cand[:n * MAXK * 2].view(n, MAXK * 2)
    K.nucleus_finish(lists, W, W * MAXK, n, sh.temp, sh.top_k, sh.top_p, sh.u, sh.out_tok, sh.ids, sh.probs, sh.keep)
    torch.cuda.synchronize()
    assert torch.equal(sh.out_tok[:n], t_full[:n])
    assert torch.equal(sh.keep[:n], full.keep[:n])
    for r in range(n):
        k = int(sh.keep[r])
        assert torch.equal(sh.ids[r, :k], full.ids[r, :k]) and torch.equal(sh.probs[r, :k], full.probs[r, :k])


def test_penalties_and_nll_match_reference():
    from velogb10_b200.engine import sampling as S
    from velogb10_b200.engine.device_sampler import DeviceSampler
    from velogb10_b200.ops import kernels as K
    v, n = 30000, 3
    x = _logits(n, v, 5, ties=False)
    hist = [[5, 7, 5, 29999, 0, 7, 7], [], [123] * 300 + list(range(200, 280))]
    params = [S.SamplingParams(0.7, 0.8, 20, 1.3, 0.5, 0.25), S.SamplingParams(0.7, 0.8, 20, 1.3, 0.5, 0.25),
              S.SamplingParams(0.0, 0.8, 20, 1.0, 1.5, 0.0)]
    ds = DeviceSampler("cuda", v, cap=16)
    assert ds.upload(params, u=[0.5] * n, histories=hist)
    y = x.clone()
    K.penalty_sharded(y, n, ds.toks, ds.cnts, ds.n_toks, ds.rep, ds.pres, ds.freq, 0)
    for r in range(n):
        ref = S.apply_penalties(x[r].cpu(), hist[r], params[r])
        assert torch.allclose(y[r].cpu(), ref, rtol=1e-6, atol=1e-6), r
    # a shard only touches its own ids
    z = x[:, 10000:20000].contiguous()
    z0 = z.clone()
    K.penalty_sharded(z, n, ds.toks, ds.cnts, ds.n_toks, ds.rep, ds.pres, ds.freq, 10000)
    assert torch.equal(z, z0)
    tgt = torch.tensor([1, 17, 29999], dtype=torch.int32, device="cuda")
    out = torch.zeros(n, device="cuda")
    K.nll(x, n, tgt, out)
    ref = -torch.log_softmax(x.double(), -1)[torch.arange(n), tgt.long()]
    assert torch.allclose(out.double(), ref, rtol=1e-5, atol=1e-5)


def test_lcg_draw_of_the_seeded_nucleus_kernel():
    from velogb10_b200.engine import sampling as S
    from velogb10_b200.ops import kernels as K
    v, n = 5000, 8
    x = _logits(n, v, 2)
    dev = "cuda"
    temp = torch.full((n,), 0.9, device=dev)
    tk = torch.full((n,), 30, dtype=torch.int32, device=dev)
    tp = torch.full((n,), 0.85, device=dev)
    seed = torch.arange(100, 100 + n, dtype=torch.int32, device=dev)
    tok = torch.zeros(n, dtype=torch.int32, device=dev)
    ids = torch.zeros(n, 64, dtype=torch.int32, device=dev)
    probs = torch.zeros(n, 64, device=dev)
    keep = torch.zeros(n, dtype=torch.int32, device=dev)
    K.nucleus(x, n, temp, tk, tp, seed, tok, ids, probs, keep)
    for r in range(n):
        k = int(keep[r])
        nuc = S.Nucleus(ids[r, :k].tolist(), probs[r, :k].tolist())
        assert int(tok[r]) == nuc.draw(S.lcg_uniform(100 + r))
        assert ids[r, :k].tolist() == S.nucleus_host(x[r].cpu(), S.SamplingParams(0.9, 0.85, 30)).ids


def test_spec_verify_matches_host_rule():
    """accept / residual resample / bonus: same (accepted, next token) as the host implementation on random nuclei,
    several lanes per launch."""
    from velogb10_b200.engine import sampling as S
    from velogb10_b200.engine.device_sampler import DeviceSampler
    rnd = random.Random(7)
    ds = DeviceSampler("cuda", 1000, cap=16)
    for trial in range(40):
        lanes, nuclei, drafts_all, keys = [], [], [], []
        col = 0
        while col < 12:
            nd = rnd.randint(0, 3)
            if col + nd + 1 > 16:
                break
            lanes.append((col, nd))
            keys.append(rnd.getrandbits(64))
            for t in range(nd + 1):
                k = rnd.randint(1, 6)
                ids = rnd.sample(range(50), k)
                pr = [rnd.random() + 0.01 for _ in range(k)]
                tot = sum(pr) * rnd.choice([1.0, 1.25])        # masses below 1 (top-p cut) as well
                nuclei.append(S.Nucleus(ids, [float(torch.tensor(x / tot, dtype=torch.float32)) for x in pr]))
                # drafts: often the top token, sometimes absent from the nucleus, sometimes its only member
                drafts_all.append(rnd.choice([ids[0], ids[-1], 77]) if t < nd else -1)
            col += nd + 1
        n = col
        ds.ids.zero_(); ds.probs.zero_()
        for c, nuc in enumerate(nuclei):
            ds.ids[c, :len(nuc.ids)] = torch.tensor(nuc.ids, dtype=torch.int32)
            ds.probs[c, :len(nuc.ids)] = torch.tensor(nuc.probs)
            ds.keep[c] = len(nuc.ids)
        u_acc, u_ver = [0.0] * n, [0.0] * n
        for (c0, nd), key in zip(lanes, keys):
            for t in range(nd + 1):
                u_acc[c0 + t] = S.rng_uniform(key, S.DOMAIN_ACCEPT, t)
                u_ver[c0 + t] = S.rng_uniform(key, S.DOMAIN_VERIFY, t)
        ds.upload([S.SamplingParams()] * n, drafts=drafts_all, u_acc=u_acc, u_ver=u_ver, lanes=lanes)
        got = ds.verify(len(lanes)).tolist()
        for (c0, nd), key, g in zip(lanes, keys, got):
            want = S.stochastic_accept(nuclei[c0:c0 + nd + 1], drafts_all[c0:c0 + nd], key)
            assert tuple(g) == want, (trial, c0, nd, g, want)

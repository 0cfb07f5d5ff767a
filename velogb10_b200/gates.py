"""Correctness gates, probes and micro-benchmarks exposed as CLI modes (``python -m velogb10_b200 --probe-binv
--synthetic tiny`` ...). Each prints one JSON line and returns 0 (pass), 1 (fail) or 2 (could not measure),
the convention the gate runner relies on.

They re-create the reference's probe modes (reference: src/main.rs:554-1232, :2036-2401; src/gpu.rs:4949-5290,
:5785-7023, :7412-7870) against this engine's runner API, so they run on the CUDA runtime and, with
``--cpu``, on the fp32 oracle. Statistical helpers (Wilson-Hilferty z, two-sample chi-square) follow
src/gpu.rs:8047-8199.
"""
from __future__ import annotations

import json
import math
import random
import time
from typing import Dict, List, Optional, Tuple

import torch

from .engine import sampling as S
from .engine.mtp import AUTO_DEPTHS, MtpPolicy
from .engine.sampling import SamplingParams
from .engine.scheduler import Request, Scheduler

GREEDY = SamplingParams(temperature=0.0)


# ------------------------------------------------------------------ statistics

def wh_z(chi2: float, dof: int) -> float:
    """Wilson-Hilferty normal approximation of a chi-square statistic."""
    if dof <= 0:
        return 0.0
    return ((chi2 / dof) ** (1.0 / 3.0) - (1.0 - 2.0 / (9.0 * dof))) / math.sqrt(2.0 / (9.0 * dof))


def two_sample_chi2(a: Dict[int, int], b: Dict[int, int], min_expected: float = 5.0) -> Tuple[float, int]:
    """Chi-square of homogeneity between two count tables; rare categories are pooled."""
    na, nb = sum(a.values()), sum(b.values())
    if na == 0 or nb == 0:
        return 0.0, 0
    keys = sorted(set(a) | set(b))
    pooled_a = pooled_b = 0
    chi2, dof = 0.0, -1
    cells = []
    for k in keys:
        ca, cb = a.get(k, 0), b.get(k, 0)
        if (ca + cb) * min(na, nb) / (na + nb) < min_expected:
            pooled_a += ca
            pooled_b += cb
        else:
            cells.append((ca, cb))
    if pooled_a + pooled_b > 0:
        cells.append((pooled_a, pooled_b))
    for ca, cb in cells:
        tot = ca + cb
        ea, eb = tot * na / (na + nb), tot * nb / (na + nb)
        if ea > 0 and eb > 0:
            chi2 += (ca - ea) ** 2 / ea + (cb - eb) ** 2 / eb
            dof += 1
    return chi2, max(dof, 0)


# ------------------------------------------------------------------ helpers

def _sync(runner):
    if hasattr(runner, "dev"):
        torch.cuda.synchronize(runner.dev)


def _rand_tokens(cfg, n: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, max(2, cfg.vocab_size - 2), (n,), generator=g).tolist()


def _snapshot(runner):
    st = runner if hasattr(runner, "S") and not hasattr(runner, "state") else None
    if st is not None:                                  # CUDA runtime
        return [t.clone() for t in (runner.S, runner.conv, runner.kc, runner.vc, getattr(runner, "ks", None), getattr(runner, "vs", None))
                if t is not None]
    s = runner.state                                    # oracle
    return [{k: v.clone() for k, v in d.items()} for d in (s.S, s.conv, s.k, s.v)]


def _restore(runner, snap):
    if hasattr(runner, "S") and not hasattr(runner, "state"):
        for t, c in zip([t for t in (runner.S, runner.conv, runner.kc, runner.vc, getattr(runner, "ks", None), getattr(runner, "vs", None))
                if t is not None], snap):
            t.copy_(c)
        return
    s = runner.state
    for d, c in zip((s.S, s.conv, s.k, s.v), snap):
        for k in d:
            d[k].copy_(c[k])


def _state_slot(runner, slot: int):
    if hasattr(runner, "S") and not hasattr(runner, "state"):
        return [runner.S[:, slot].clone(), runner.conv[:, slot].clone()]
    s = runner.state
    return [torch.stack([s.S[k][slot] for k in sorted(s.S)]), torch.stack([s.conv[k][slot] for k in sorted(s.conv)])]


def _emit(name: str, ok: bool, **kw) -> int:
    print(json.dumps({"gate": name, "pass": bool(ok), **kw}))
    return 0 if ok else 1


# ------------------------------------------------------------------ gates

def gate_verify_fuzz(runner, cfg, draws: int = 8, seed: int = 0, max_seq: int = 1200) -> int:
    """verify(N) == N sequential decodes (logits bits and state) at random (context, depth), with contexts
    chosen around multiples of the 256-key attention split."""
    rng = random.Random(seed)
    offs = [0, 250, 254, 255, 256, 510, 511, 1022, 1023]
    bad = 0
    for d in range(draws):
        depth = rng.choice([2, 3, 4, 6, 8])
        ctx = min(max_seq - depth - 2, max(4, rng.choice(offs) + rng.randint(0, 3)))
        toks = _rand_tokens(cfg, ctx + depth, seed * 1000 + d)
        runner.zero_slot(0)
        runner.prefill(0, toks[:ctx], 0)
        snap = _snapshot(runner)
        lv, _ = runner.verify(0, toks[ctx:], ctx, ckpt_base=1)
        lv = lv.clone()
        ck = [_state_slot(runner, 1 + t) for t in range(depth)]
        _restore(runner, snap)
        for t in range(depth):
            ld, _ = runner.decode([toks[ctx + t]], [ctx + t], [0])
            st = _state_slot(runner, 0)
            if not torch.equal(ld[0], lv[t]) or not all(torch.equal(a, b) for a, b in zip(st, ck[t])):
                bad += 1
                break
    return _emit("verify-fuzz", bad == 0, draws=draws, failures=bad, seed=seed)


def gate_state(runner, cfg) -> int:
    """After verify + rollback to an accepted prefix, recurrent state and later logits equal pure decode."""
    ctx, depth, nacc = 40, 6, 3
    toks = _rand_tokens(cfg, ctx + depth + 1, 7)
    runner.zero_slot(0)
    runner.prefill(0, toks[:ctx], 0)
    snap = _snapshot(runner)
    runner.verify(0, toks[ctx:ctx + depth], ctx, ckpt_base=1)
    runner.copy_state(1 + nacc - 1, 0)                         # keep the first nacc columns
    la, _ = runner.decode([toks[ctx + nacc]], [ctx + nacc], [0])
    la = la.clone()
    sa = _state_slot(runner, 0)
    _restore(runner, snap)
    for t in range(nacc):
        runner.decode([toks[ctx + t]], [ctx + t], [0])
    lb, _ = runner.decode([toks[ctx + nacc]], [ctx + nacc], [0])
    ok = torch.equal(la, lb) and all(torch.equal(a, b) for a, b in zip(sa, _state_slot(runner, 0)))
    return _emit("state", ok)


def gate_binv(runner, cfg) -> int:
    """Every GEMM site: column 0 at widths 1..16 has the bits of width 1; result close to the dequantised
    reference (CUDA runtime only)."""
    if not hasattr(runner, "dev"):
        return _emit("binv", True, note="oracle computes every column independently")
    from .ops import gemm as G
    worst, sites, bad = 0.0, 0, []
    for name, q in runner.w.linears():
        if q.kernel is None or q.experts > 1 or sites >= 12:
            continue
        sites += 1
        x = (torch.randn(16, q.k, device=runner.dev) * 0.5).to(torch.float16)
        base = G.linear(q, x, 1, out_f32=True)[0].clone()
        for n in range(2, 17):
            if not torch.equal(G.linear(q, x, n, out_f32=True)[0], base):
                bad.append((name, n))
                break
        if q.packed is not None or q.codes is not None or q.w is not None:
            ref = x[:1].float() @ q.dequant(torch.float32).t()
            worst = max(worst, float((base - ref[0]).norm() / ref.norm().clamp(min=1e-9)))
    return _emit("binv", not bad and worst < 0.01, sites=sites, mismatches=bad[:4], rel_l2=worst)


def _stream(runner, cfg, prompt, n_new, policy, params=GREEDY, max_seq=512, **kw):
    sch = Scheduler(runner, 1, max_seq, eos_ids=[], policy=policy, **kw)
    out: List[int] = []
    t0 = time.time()
    sch.submit(Request(prompt, n_new, params, on_token=out.append))
    sch.run_until_idle()
    _sync(runner)
    return out, time.time() - t0, sch


def gate_mtp_lossless(runner, cfg, n_new: int = 48, depth: int = 4, **kw) -> int:
    if runner.w.mtp is None:
        return _emit("mtp-lossless", False, error="model has no MTP head") or 2
    prompt = _rand_tokens(cfg, 24, 3)
    base, tb, _ = _stream(runner, cfg, prompt, n_new, MtpPolicy("off", has_head=True))
    spec, ts, sch = _stream(runner, cfg, prompt, n_new, MtpPolicy("on", depth=depth), **kw)
    ok = base == spec and len(spec) == n_new
    return _emit("mtp-lossless", ok, LOSSLESS_OK=ok, acceptance=sch.policy.acceptance(), tok_s_plain=n_new / tb,
                 tok_s_mtp=n_new / ts, mtp_steps=sch.stats["mtp_steps"])


def gate_tree(runner, cfg) -> int:
    """Twin-branch equality and random tree vs per-path chain oracle. Runs the runner as a tree-drafting scheduler
    does: every attention call through the path-indirect kernel (the tensor-core decode kernel has no path form, and
    two kernels do not round alike)."""
    tc = getattr(runner, "tc_decode_attn", None)
    if tc is not None:
        runner.tc_decode_attn = False
    try:
        return _gate_tree(runner, cfg)
    finally:
        if tc is not None:
            runner.tc_decode_attn = tc


def _gate_tree(runner, cfg) -> int:
    ctx = 30
    toks = _rand_tokens(cfg, ctx, 11)
    runner.zero_slot(0)
    runner.prefill(0, toks, 0)
    snap = _snapshot(runner)
    cols = [5, 6, 7, 6, 7]                       # root, A = (6, 7), B = (6, 7): twin branches
    parent = [-1, 0, 1, 0, 3]
    lt, _ = runner.verify(0, cols, ctx, ckpt_base=1, parent=parent)
    lt = lt.clone()
    twin = torch.equal(lt[1], lt[3]) and torch.equal(lt[2], lt[4])
    _restore(runner, snap)
    lc, _ = runner.verify(0, cols[:3], ctx, ckpt_base=1)
    chain = all(torch.equal(lc[i], lt[i]) for i in range(3))
    return _emit("tree", twin and chain, twin=twin, chain=chain)


def gate_lanes(runner, cfg) -> int:
    """A packed forest verify gives each lane the logits it gets alone (lengths around the 256 boundary)."""
    lens = [250, 257]
    seqs = [_rand_tokens(cfg, l + 3, 20 + i) for i, l in enumerate(lens)]
    for s, (l, sq) in enumerate(zip(lens, seqs)):
        runner.zero_slot(s)
        runner.prefill(s, sq[:l], 0)
    snap = _snapshot(runner)
    alone = []
    for s, (l, sq) in enumerate(zip(lens, seqs)):
        lv, _ = runner.verify(s, sq[l:], l, ckpt_base=2 + 4 * s)
        alone.append(lv.clone())
    _restore(runner, snap)
    packed = runner.verify_forest([(s, sq[l:], l, 2 + 4 * s) for s, (l, sq) in enumerate(zip(lens, seqs))])
    ok = all(torch.equal(a, p[0]) for a, p in zip(alone, packed))
    return _emit("lanes", ok)


def gate_mtp_sample(runner, cfg, trials: int = 400, temp: float = 0.7) -> int:
    """Stochastic speculation emits the plain sampler's distribution: two-sample chi-square on the first
    emitted tokens over many seeds, |z| < 4."""
    if runner.w.mtp is None:
        return 2
    prompt = _rand_tokens(cfg, 16, 5)
    plain: Dict[int, int] = {}
    spec: Dict[int, int] = {}
    for t in range(trials):
        sp = SamplingParams(temperature=temp, top_p=0.95, top_k=16, seed=1000 + t)
        a, _, _ = _stream(runner, cfg, prompt, 3, MtpPolicy("off", has_head=True), sp, max_seq=64)
        b, _, _ = _stream(runner, cfg, prompt, 3, MtpPolicy("on", depth=3), sp, max_seq=64)
        plain[a[1]] = plain.get(a[1], 0) + 1
        spec[b[1]] = spec.get(b[1], 0) + 1
    chi2, dof = two_sample_chi2(plain, spec)
    z = wh_z(chi2, dof)
    return _emit("mtp-sample", abs(z) < 4.0, z=z, chi2=chi2, dof=dof, trials=trials)


# ------------------------------------------------------------------ benches / probes

def calibrate_mtp_r(runner, sched: Optional[Scheduler] = None, steps: int = 8) -> Dict[int, float]:
    """Cost ratio r(d) of one speculative step (draft + verify + rollback + reprime) over one decode step."""
    cfg = runner.cfg
    ctx = 64
    toks = _rand_tokens(cfg, ctx + 32, 9)
    runner.zero_slot(0)
    _, hidden = runner.prefill(0, toks[:ctx], 0)

    def timed(fn):
        fn()
        _sync(runner)
        t0 = time.perf_counter()
        for _ in range(steps):
            fn()
        _sync(runner)
        return (time.perf_counter() - t0) / steps

    # what the scheduler runs: graph replays of the decode step and of the chain verify where the runner has them
    graphs = hasattr(runner, "replay_decode") and hasattr(runner, "replay_verify") and (sched is None or sched.use_graphs)
    if graphs:
        base = timed(lambda: runner.replay_decode([toks[ctx]], [ctx], [0]))
    else:
        base = timed(lambda: runner.decode([toks[ctx]], [ctx], [0]))
    table = {}
    h = hidden[-1:].clone()
    for d in AUTO_DEPTHS:
        def step():
            for j in range(d - 1):
                runner.mtp_forward(0, [toks[ctx + j]], h, [ctx - 1 + j])
            if graphs:
                _, hid = runner.replay_verify(0, toks[ctx:ctx + d], ctx, 1)
            else:
                _, hid = runner.verify(0, toks[ctx:ctx + d], ctx, ckpt_base=1)
            hid = hid.clone()
            runner.copy_state(1, 0)
            runner.mtp_forward(0, toks[ctx + 1:ctx + d], hid[:d - 1], list(range(ctx, ctx + d - 1)))
        table[d] = timed(step) / base
    return table


def bench_prefill(runner, cfg, n: int = 1024) -> int:
    toks = _rand_tokens(cfg, n, 1)
    runner.zero_slot(0)
    runner.prefill(0, toks[:min(64, n)], 0)
    runner.zero_slot(0)
    _sync(runner)
    t0 = time.perf_counter()
    runner.prefill(0, toks, 0)
    _sync(runner)
    dt = time.perf_counter() - t0
    return _emit("bench-prefill", True, tokens=n, ms=dt * 1e3, tok_s=n / dt)


def bench_batch(runner, cfg, batch: int = 4, steps: int = 16) -> int:
    for s in range(batch):
        runner.zero_slot(s)
        runner.prefill(s, _rand_tokens(cfg, 32 + s, s), 0)
    toks, pos = [1] * batch, [32 + s for s in range(batch)]
    runner.decode(toks, pos, list(range(batch)))
    _sync(runner)
    t0 = time.perf_counter()
    for i in range(steps):
        runner.decode(toks, [p + 1 + i for p in pos], list(range(batch)))
    _sync(runner)
    dt = time.perf_counter() - t0
    return _emit("bench-batch", True, batch=batch, ms_per_step=dt / steps * 1e3, tok_s=batch * steps / dt)


def perplexity(runner, cfg, n: int = 128) -> int:
    """Mean NLL of a token stream under the model (synthetic ids unless a corpus file is given)."""
    toks = _rand_tokens(cfg, n, 17)
    runner.zero_slot(0)
    nll = 0.0
    for t in range(n - 1):
        lg, _ = runner.decode([toks[t]], [t], [0])
        lp = torch.log_softmax(lg[0].float(), -1)
        nll -= float(lp[toks[t + 1]])
    return _emit("perplexity", True, tokens=n - 1, nll=nll / (n - 1), ppl=math.exp(nll / (n - 1)))


def probe_bandwidth(runner, sustained: bool = False) -> int:
    if not hasattr(runner, "dev"):
        return 2
    n = 1 << 28
    a = torch.empty(n, dtype=torch.float32, device=runner.dev)
    b = torch.empty_like(a)
    best, t_end = 0.0, time.time() + (4.0 if sustained else 0.0)
    samples = []
    while True:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        b.copy_(a)
        e1.record()
        torch.cuda.synchronize()
        gbs = 2 * n * 4 / (e0.elapsed_time(e1) * 1e6)
        samples.append(gbs)
        best = max(best, gbs)
        if len(samples) >= 10 and time.time() > t_end:
            break
    return _emit("probe-bandwidth", True, copy_GBs_best=best, copy_GBs_last=samples[-1], samples=len(samples))


def probe_gemm(runner, cfg, sweep: bool = False) -> int:
    if not hasattr(runner, "dev"):
        return 2
    from .ops import gemm as G
    rows = []
    for name, q in runner.w.linears():
        if q.kernel is None or q.experts > 1:
            continue
        x = (torch.randn(16, q.k, device=runner.dev) * 0.5).to(torch.float16)
        for n in ([1, 2, 4, 8, 16] if sweep else [1]):
            G.linear(q, x, n)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(5):
                G.linear(q, x, n)
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 200
            rows.append({"site": name, "m": q.m, "k": q.k, "n": n, "us": us,
                         "GBs": q.kernel.wt.numel() / us / 1e3})
        if len(rows) >= (40 if sweep else 12):
            break
    return _emit("probe-gemm", True, rows=rows)


def probe_moe(runner, cfg) -> int:
    """Dump one MoE block's routing and output for an external oracle."""
    lay = next((l for l in runner.w.layers if l.moe is not None), None)
    if lay is None:
        return 2
    toks = _rand_tokens(cfg, 4, 2)
    runner.zero_slot(0)
    lg, hid = runner.prefill(0, toks, 0)
    return _emit("probe-moe", True, tokens=toks, hidden_norm=float(hid.float().norm()), argmax=int(lg.argmax()))


def capture_layers(runner, cfg) -> int:
    toks = _rand_tokens(cfg, 8, 4)
    runner.zero_slot(0)
    lg, hid = runner.prefill(0, toks, 0)
    return _emit("capture-layers", True, tokens=toks, final_hidden_absmax=float(hid.float().abs().max()),
                 logits_absmax=float(lg.float().abs().max()), argmax=int(lg.argmax()))


def dump_argmax(runner, cfg, n: int = 16) -> int:
    out, _, _ = _stream(runner, cfg, _rand_tokens(cfg, 12, 6), n, MtpPolicy("off", has_head=runner.w.mtp is not None))
    print("GATE_TOKENS " + " ".join(str(t) for t in out))
    return _emit("dump-argmax", len(out) == n, tokens=out)


def profile_mtp(runner, cfg) -> int:
    if runner.w.mtp is None:
        return 2
    return _emit("profile-mtp", True, r={str(k): v for k, v in calibrate_mtp_r(runner).items()})


def tp_barrier_bench(args) -> int:
    """Adversarial loop over the peer-memory transport (run under torchrun): many epochs of every collective path with
    payloads that name their epoch, checked ON THE DEVICE every epoch, random host-side stalls on one rank, and the
    requirement of zero validation errors and zero timeouts (reference: src/tp_bench.rs:158-324). Paths (``--paths``):

    * ``allreduce``  the stand-alone one-shot all-reduce kernel;
    * ``fused``      the decode-width form used by the model: row-parallel FP4 GEMM whose epilogue publishes its partial
                     rows + the residual-add / RMSNorm kernel that sums the ranks (pair push or in-switch reduction,
                     whichever the communicator selected);
    * ``gemm_rs``    prefill-width GEMM fused with the reduce-scatter + its finish kernel;
    * ``ag_gemm``    all-gather pushes + flag-gated GEMM.

    Inputs are scaled by 2^(epoch mod 8): every stage (FP4 series, GEMM, bf16 rounding) commutes exactly with a power
    of two, so the expected output of epoch e is a precomputed reference times that factor and equality is exact. A
    stale or torn read shows up as a mismatch because consecutive uses of a buffer set carry different factors."""
    import os
    import random
    import torch.distributed as dist
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    if world < 2:
        return _emit("tp-barrier-bench", False, error="run under torchrun with >= 2 ranks") or 2
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    from .models.weights import QLinear
    from .ops import gemm as G
    from .parallel.comm import TpComm
    comm = TpComm(rank, world, dev, max_elems=1 << 22, ag_bytes=2 * 512 * 1024 * 2 * 2)
    paths = args.get("--paths", "allreduce,fused,gemm_rs,ag_gemm").split(",")
    epochs = int(float(args.get("--epochs", "1000000")))
    heavy_epochs = int(float(args.get("--heavy-epochs", str(max(1000, epochs // 50)))))
    stall = rank == world - 1 and args.get("--stall", "on") != "off"
    rnd = random.Random(1234)
    gw = torch.Generator(device=dev).manual_seed(7)
    h, kloc = 5120, 1024
    results = {}
    status_failed = False

    def maybe_stall(e):
        if stall and e % 997 == 0:
            time.sleep(rnd.random() * (0.005 if e % 49850 == 0 else 0.0003))

    def finish(name, n_ep, err_dev, t0):
        nonlocal status_failed
        torch.cuda.synchronize()
        dt = time.time() - t0
        timeouts = 0
        try:
            comm.check()
        except Exception:  # noqa: BLE001
            timeouts = 1
            status_failed = True
        results[name] = {"epochs": n_ep, "validation_errors": int(err_dev.item()), "timeouts": timeouts,
                         "us_per_epoch": dt / max(n_ep, 1) * 1e6}
        dist.barrier()

    scales = [float(2 ** i) for i in range(8)]
    if "allreduce" in paths:
        err = torch.zeros((), dtype=torch.int64, device=dev)
        base = torch.arange(5120, device=dev, dtype=torch.float32).remainder(61).add_(rank + 1).reshape(1, -1)
        want = sum((torch.arange(5120, device=dev, dtype=torch.float32).remainder(61) + q + 1) for q in range(world)).reshape(1, -1)
        ins = [base * s_ for s_ in scales]
        wants = [want * s_ for s_ in scales]
        buf = torch.empty_like(base)
        t0 = time.time()
        for e in range(epochs):
            maybe_stall(e)
            buf.copy_(ins[e % 8])
            comm.all_reduce_rows(buf, 1)
            err += (buf != wants[e % 8]).any()
        finish("allreduce", epochs, err, t0)
    if "fused" in paths:
        wf = (torch.randn(h, kloc * world, generator=gw, device=dev) * 0.05).to(torch.bfloat16)
        xa = torch.randn(16, kloc * world, generator=gw, device=dev).to(torch.float16)
        q = QLinear.from_dense(wf[:, rank * kloc:(rank + 1) * kloc].contiguous(), "nvfp4")
        x_loc = [(xa[:, rank * kloc:(rank + 1) * kloc] * s_).contiguous() for s_ in scales]
        acts = []
        for xs in x_loc:                                  # private quantised copies: the loop then only runs the fused pair
            bq, sfb, g0 = G.quantize_act_fp4(xs, 4, q.kernel4.kp if getattr(q, "kernel4", None) else G.prepare_fp4(q).kp)
            acts.append((bq.clone(), sfb.clone(), g0.clone()))
        ones = torch.zeros(h, device=dev)
        x16 = torch.zeros(16, h, dtype=torch.float16, device=dev)
        dummy = torch.zeros(16, h, dtype=torch.bfloat16, device=dev)
        mode = 2 if comm.use_mm else 1
        res = torch.zeros(16, h, dtype=torch.bfloat16, device=dev)
        refs = []
        for i in range(8):                                # reference = what the path itself produces once, then it must repeat
            res.zero_()
            G.linear_fp4(q, x_loc[i], 4, out=dummy, comm=comm, act=acts[i], push_only=True)
            G.add_rmsnorm_fp4_ar(res, ones, 1e-6, 4, comm, out16=x16, mode=mode)
            refs.append(res[:4].clone())
        torch.cuda.synchronize()
        exact_scaling = all(torch.equal(refs[i], refs[0] * scales[i]) for i in range(8))
        err = torch.zeros((), dtype=torch.int64, device=dev)
        t0 = time.time()
        for e in range(epochs):
            maybe_stall(e)
            res.zero_()
            G.linear_fp4(q, x_loc[e % 8], 4, out=dummy, comm=comm, act=acts[e % 8], push_only=True)
            G.add_rmsnorm_fp4_ar(res, ones, 1e-6, 4, comm, out16=x16, mode=mode)
            err += (res[:4] != refs[e % 8]).any()
        finish("fused", epochs, err, t0)
        results["fused"]["power_of_two_scaling_exact"] = bool(exact_scaling)
        results["fused"]["form"] = "in-switch multimem.ld_reduce" if comm.use_mm else "(value, epoch) pair push"
    if "gemm_rs" in paths:
        n_tok, M_, K_ = 256 * world, 1024, 1024
        w = (torch.randn(M_, K_ * world, generator=gw, device=dev) * 0.05).to(torch.bfloat16)
        xf = torch.randn(n_tok, K_ * world, generator=gw, device=dev).to(torch.float16)
        q = QLinear.from_dense(w[:, rank * K_:(rank + 1) * K_].contiguous(), "nvfp4")
        G.prepare(q)
        xs = [(xf[:, rank * K_:(rank + 1) * K_] * s_).contiguous() for s_ in scales]
        out = torch.zeros(n_tok, M_, dtype=torch.bfloat16, device=dev)
        rs_rows = comm.rs_rows_for(n_tok, M_)
        refs = []
        for i in range(8):
            G.linear(q, xs[i], n_tok, out=out, comm=comm, rs_rows=rs_rows)
            comm.gemm_rs_finish(out, n_tok, rs_rows)
            refs.append(out.clone())
        err = torch.zeros((), dtype=torch.int64, device=dev)
        t0 = time.time()
        for e in range(heavy_epochs):
            maybe_stall(e * 50)
            G.linear(q, xs[e % 8], n_tok, out=out, comm=comm, rs_rows=rs_rows)
            comm.gemm_rs_finish(out, n_tok, rs_rows)
            err += (out != refs[e % 8]).any()
        finish("gemm_rs", heavy_epochs, err, t0)
    if "ag_gemm" in paths:
        rows_per, K_, M_ = 128, 1024, 512
        n_total = rows_per * world
        w = (torch.randn(M_, K_, generator=gw, device=dev) * 0.05).to(torch.bfloat16)
        xf = torch.randn(n_total, K_, generator=gw, device=dev).to(torch.float16)
        q = QLinear.from_dense(w, "nvfp4")
        shards = [(xf[rank * rows_per:(rank + 1) * rows_per] * s_).contiguous() for s_ in scales]
        out = torch.zeros(n_total, M_, dtype=torch.bfloat16, device=dev)
        refs = []
        for i in range(8):
            comm.ag_gemm(q, shards[i], rank * rows_per, n_total, out)
            refs.append(out.clone())
        err = torch.zeros((), dtype=torch.int64, device=dev)
        t0 = time.time()
        for e in range(heavy_epochs):
            maybe_stall(e * 50)
            comm.ag_gemm(q, shards[e % 8], rank * rows_per, n_total, out)
            err += (out != refs[e % 8]).any()
        finish("ag_gemm", heavy_epochs, err, t0)
    ok = all(r["validation_errors"] == 0 and r["timeouts"] == 0 for r in results.values()) and not status_failed
    # every rank must have seen a clean run
    flag = torch.tensor([0 if ok else 1], device=dev)
    dist.all_reduce(flag)
    ok = int(flag.item()) == 0
    if rank == 0:
        _emit("tp-barrier-bench", ok, world=world, stalls_injected=bool(args.get("--stall", "on") != "off"),
              arena=comm.describe()["arena"], **results)
    dist.barrier()
    return 0 if ok else 1


# ------------------------------------------------------------------ dispatch

def dispatch(args: Dict[str, str]) -> int:
    from .cli import load_runner
    if "--tp-barrier-bench" in args or "--net-test" in args:
        return tp_barrier_bench(args)
    modes = [m for m in ("--probe-binv", "--bench-verify", "--probe-state", "--probe-reject", "--bench-mtp",
                         "--bench-mtp-sample", "--bench-tree", "--bench-lanes", "--bench-accept", "--bench-prefill",
                         "--bench-batch", "--profile-mtp", "--perplexity", "--probe-bandwidth",
                         "--probe-bandwidth-sustained", "--probe-gemm", "--sweep-gemm", "--probe-tp-gemv", "--probe-moe",
                         "--capture-layers", "--dump-argmax") if m in args]
    if not modes:
        print(json.dumps({"error": "no mode given; see --help"}))
        return 2
    max_seq = int(args.get("--max-seq-len", "1280"))
    runner, tok, cfg, max_seq = load_runner(args, 4, max_seq)
    runner.alloc_state(4, 4 + 17 + 4, max_seq)
    rc = 0
    for m in modes:
        if hasattr(runner, "n_slots") and (runner.n_slots != 4 or runner.max_seq != max_seq):
            runner.alloc_state(4, 4 + 17 + 4, max_seq)     # a gate that ran a scheduler re-sized the state for itself
        if m == "--probe-binv":
            r = gate_binv(runner, cfg)
        elif m == "--bench-verify":
            r = gate_verify_fuzz(runner, cfg, int(args.get("--draws", "6")), int(args.get("--seed", "0")), max_seq)
        elif m in ("--probe-state", "--probe-reject"):
            r = gate_state(runner, cfg)
        elif m in ("--bench-mtp", "--bench-accept"):
            r = gate_mtp_lossless(runner, cfg, int(args.get("--max-new", "48")), int(args.get("--mtp-depth", "4")))
        elif m == "--bench-mtp-sample":
            r = gate_mtp_sample(runner, cfg, int(args.get("--trials", "400")))
        elif m == "--bench-tree":
            r = gate_tree(runner, cfg)
        elif m == "--bench-lanes":
            r = gate_lanes(runner, cfg)
        elif m == "--bench-prefill":
            r = bench_prefill(runner, cfg, int(args.get("--tokens", "1024")))
        elif m == "--bench-batch":
            r = bench_batch(runner, cfg, int(args.get("--batch", "4")))
        elif m == "--profile-mtp":
            r = profile_mtp(runner, cfg)
        elif m == "--perplexity":
            r = perplexity(runner, cfg, int(args.get("--tokens", "128")))
        elif m in ("--probe-bandwidth", "--probe-bandwidth-sustained"):
            r = probe_bandwidth(runner, m.endswith("sustained"))
        elif m in ("--probe-gemm", "--sweep-gemm", "--probe-tp-gemv"):
            r = probe_gemm(runner, cfg, m == "--sweep-gemm")
        elif m == "--probe-moe":
            r = probe_moe(runner, cfg)
        elif m == "--capture-layers":
            r = capture_layers(runner, cfg)
        else:
            r = dump_argmax(runner, cfg)
        rc = max(rc, r)
    return rc

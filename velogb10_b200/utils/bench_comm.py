"""Fused compute + collective paths against their library (NCCL) baselines at the model's real message shapes, one
process per GPU under torchrun. For every path: CUDA-event time per call (maximum over ranks), a per-call latency
histogram, and the achieved fraction of the path's roofline = the slower of (FLOPs / measured bf16 GEMM peak) and
(bytes that must cross NVLink per GPU / measured 770 GB/s per direction), plus the weight-streaming bound for the
decode-width GEMMs, whose floor is HBM, not NVLink.

  python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \\
      -m velogb10_b200.utils.bench_comm --iters 200

Paths:
  decode_allreduce   row-parallel FP4 GEMM [h x K/W] whose epilogue publishes partial rows + residual-add / RMSNorm
                     consumer (pair push and, when the arena is multicast-bound, in-switch multimem.ld_reduce)
                     vs the same GEMM + dist.all_reduce + the plain norm kernel
  gemm_rs            prefill-width GEMM fused with the reduce-scatter + finish kernel vs GEMM + dist.all_reduce
  ag_gemm            all-gather pushes + flag-gated GEMM vs dist.all_gather_into_tensor + GEMM
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0          # measured peer copy, per direction per GPU
HBM_GBS = 6540.8
BF16_TFLOPS = 1396.3        # measured sustained cuBLAS bf16


def _peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        d = json.load(open(p))
        return float(d["hbm_gbs"]), float(d["bf16_tflops_sustained"])
    except Exception:  # noqa: BLE001 - file absent: the recorded values above
        return HBM_GBS, BF16_TFLOPS


def timed(fn, iters, warm=5):
    """Per-call device times (us) of ``iters`` calls, each bracketed by its own events after a barrier-free warm-up."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for a, b in evs:
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    return [a.elapsed_time(b) * 1e3 for a, b in evs]


def summary(us, world):
    t = torch.tensor(us, dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)             # a collective is as slow as its slowest rank
    v = sorted(t.tolist())
    pick = lambda q: v[min(len(v) - 1, int(q * len(v)))]
    edges = [0, 5, 10, 15, 20, 30, 50, 100, 200, 500, 1e9]
    hist = {f"<{int(hi)}us" if hi < 1e9 else ">=500us": sum(1 for x in v if lo <= x < hi) for lo, hi in zip(edges[:-1], edges[1:])}
    return {"p50_us": round(pick(0.5), 2), "p90_us": round(pick(0.9), 2), "p99_us": round(pick(0.99), 2), "max_us": round(v[-1], 2),
            "hist": {k: c for k, c in hist.items() if c}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=200)
    ap.add_argument("--hidden", type=int, default=5120)
    ap.add_argument("--inter", type=int, default=17408)
    ap.add_argument("--tokens", type=int, default=4096)
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from ..models.weights import QLinear
    from ..ops import gemm as G, kernels as K, lib as vlib
    from ..parallel.comm import TpComm
    hbm, tfl = _peaks()
    h, I = args.hidden, args.inter
    comm = TpComm(rank, world, dev, ag_bytes=2 * args.tokens * h * 2 * 2)
    g = torch.Generator(device=dev).manual_seed(3 + rank)
    rows = []

    # ---------------------------------------------------------------- decode-width all-reduce (down projection shape)
    kloc = (I // world + 255) // 256 * 256
    q = QLinear.from_dense((torch.randn(h, kloc, generator=g, device=dev) * 0.02).to(torch.bfloat16), "nvfp4")
    x = torch.randn(16, kloc, generator=g, device=dev).to(torch.float16)
    res = torch.zeros(16, h, dtype=torch.bfloat16, device=dev)
    x16 = torch.zeros(16, h, dtype=torch.float16, device=dev)
    wn = torch.zeros(h, device=dev)
    out = torch.zeros(16, h, dtype=torch.bfloat16, device=dev)
    wbytes = h * kloc // 2 * 1.125
    for n in (1, 4, 16):
        act = G.quantize_act_fp4(x, n, G.prepare_fp4(q).kp)
        act = tuple(t.clone() for t in act)
        forms = [("pair_push", 1)] + ([("multimem_ld_reduce", 2)] if comm.mc else [])
        for name, mode in forms:
            comm.use_mm = mode == 2

            def fused():
                G.linear_fp4(q, x, n, out=out, comm=comm, act=act, push_only=True)
                G.add_rmsnorm_fp4_ar(res, wn, 1e-6, n, comm, out16=x16, mode=mode)
            us = timed(fused, args.iters)
            s_ = summary(us, world)
            floor_us = max(wbytes / hbm / 1e3, n * h * 4 * (world - 1) / world / NVLINK_GBS / 1e3)
            rows.append({"path": "decode_allreduce", "form": name, "cols": n, "shape": [h, kloc], **s_,
                         "roofline_us": round(floor_us, 2), "fraction_of_roofline": round(floor_us / s_["p50_us"], 3)})

        def nccl():
            G.linear_fp4(q, x, n, out=out, act=act)
            dist.all_reduce(out[:n])
            G.add_rmsnorm_fp4(res, out, wn, 1e-6, n, out16=x16)
        s_ = summary(timed(nccl, args.iters), world)
        rows.append({"path": "decode_allreduce", "form": "nccl_all_reduce + norm", "cols": n, "shape": [h, kloc], **s_})
    comm.use_mm = bool(comm.mc) and world >= int(os.environ.get("VELO_MULTIMEM_MIN_WORLD", "4"))

    # ---------------------------------------------------------------- prefill-width GEMM + reduce-scatter
    n_tok = args.tokens
    G.prepare(q)
    xs = torch.randn(n_tok, kloc, generator=g, device=dev).to(torch.float16)
    o2 = torch.zeros(n_tok, h, dtype=torch.bfloat16, device=dev)
    rs_rows = comm.rs_rows_for(n_tok, h)
    if rs_rows:
        def fused_rs():
            G.linear(q, xs, n_tok, out=o2, comm=comm, rs_rows=rs_rows)
            comm.gemm_rs_finish(o2, n_tok, rs_rows)

        def nccl_rs():
            G.linear(q, xs, n_tok, out=o2)
            dist.all_reduce(o2)
        flops = 2.0 * n_tok * h * kloc
        link_bytes = n_tok * h * 4 * (world - 1) / world + n_tok * h * 2 * (world - 1) / world     # fp32 partials out, bf16 result back
        floor_us = max(flops / tfl / 1e6, link_bytes / NVLINK_GBS / 1e3)
        forms = [("gemm + reduce-scatter fused, finish kernel", fused_rs), ("gemm + nccl_all_reduce", nccl_rs)]
        sb = comm.symmetric_buffer(n_tok * h * 2)
        if sb is not None:
            o_mm = sb.view(torch.bfloat16).view(n_tok, h)

            def mm_rs():
                G.linear(q, xs, n_tok, out=o_mm)
                comm.all_reduce_multimem(o_mm, n_tok)
            forms.insert(0, ("gemm + in-switch multimem all-reduce (in place)", mm_rs))
        for name, fn in forms:
            s_ = summary(timed(fn, max(20, args.iters // 5)), world)
            rows.append({"path": "gemm_rs", "form": name, "tokens": n_tok, "shape": [h, kloc], **s_, "roofline_us": round(floor_us, 1),
                         "fraction_of_roofline": round(floor_us / s_["p50_us"], 3)})

    # ---------------------------------------------------------------- all-gather + GEMM (gate_up shape, token rows sharded)
    mloc = (2 * I // world + 127) // 128 * 128
    qg = QLinear.from_dense((torch.randn(mloc, h, generator=g, device=dev) * 0.02).to(torch.bfloat16), "nvfp4")
    G.prepare(qg)
    rows_per = (n_tok // world + 127) // 128 * 128
    n_total = rows_per * world
    shard = torch.randn(rows_per, h, generator=g, device=dev).to(torch.float16)
    full = torch.zeros(n_total, h, dtype=torch.float16, device=dev)
    o3 = torch.zeros(n_total, mloc, dtype=torch.bfloat16, device=dev)

    def fused_ag():
        comm.ag_gemm(qg, shard, rank * rows_per, n_total, o3)

    def nccl_ag():
        dist.all_gather_into_tensor(full, shard)
        G.linear(qg, full, n_total, out=o3)
    flops = 2.0 * n_total * mloc * h
    link_bytes = rows_per * h * 2 * (world - 1)
    floor_us = max(flops / tfl / 1e6, link_bytes / NVLINK_GBS / 1e3)
    for name, fn in (("all-gather pushes + flag-gated gemm", fused_ag), ("nccl_all_gather + gemm", nccl_ag)):
        s_ = summary(timed(fn, max(20, args.iters // 5)), world)
        rows.append({"path": "ag_gemm", "form": name, "tokens": n_total, "shape": [mloc, h], **s_, "roofline_us": round(floor_us, 1),
                     "fraction_of_roofline": round(floor_us / s_["p50_us"], 3)})
    torch.cuda.synchronize()
    comm.check()
    vlib.check_err_word(dev)
    if rank == 0:
        for r in rows:
            print(json.dumps(r))
        print(json.dumps({"bench": "fused collectives vs library", "world": world, "arena": comm.describe()["arena"],
                          "peaks": {"hbm_gbs": hbm, "bf16_tflops_sustained": tfl, "nvlink_gbs_per_direction": NVLINK_GBS}}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

"""Micro-benchmark of the tensor-core GEMM on decode / prefill shapes.

  python -m velogb10_b200.utils.bench_gemm --shapes 27b --n 1

Weights are replicated until the working set exceeds L2 and the copies are cycled between timed launches,
so every launch streams its weights from HBM. Time is measured with CUDA events after warm-up; the
achieved bandwidth counts the packed weight bytes only.
"""
from __future__ import annotations

import argparse
import json

import torch

SHAPES = {
    "27b": [("gdn_in", 16480, 5120), ("gdn_out", 5120, 6144), ("gate_up", 34816, 5120), ("down", 5120, 17408),
            ("qkv", 14336, 5120), ("lm_head", 248320, 5120)],
    "35b": [("gdn_in", 12352, 2048), ("out", 2048, 4096), ("qkv", 9216, 2048), ("lm_head", 248320, 2048)],
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="27b")
    ap.add_argument("--n", type=int, default=1)
    ap.add_argument("--fmt", default="nvfp4")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--splitk", default="auto")
    ap.add_argument("--only", default="")
    ap.add_argument("--fp4", action="store_true", help="time the block-scaled FP4 path (nvfp4 weights, N <= 16)")
    args = ap.parse_args()
    from ..models.weights import QLinear
    from ..ops import gemm as G, lib as vlib
    L = vlib.lib()
    for name, m, k in SHAPES[args.shapes]:
        if args.only and name not in args.only.split(","):
            continue
        w = (torch.randn(min(m, 8192), k, device="cuda") * 0.02).to(torch.bfloat16)
        w = w.repeat((m + w.shape[0] - 1) // w.shape[0], 1)[:m].contiguous()
        q = QLinear.from_dense(w, args.fmt)
        del w
        bytes_w = q.nbytes() - (q.row_scale.numel() * 4 if q.row_scale is not None else 0)
        copies = max(2, int(300e6 // bytes_w) + 1) if bytes_w < 300e6 else 2
        tws = []
        for c in range(copies):
            qc = QLinear(q.fmt, q.m, q.k, q.packed, q.scales, q.codes, q.row_scale, q.w)
            tw = G.prepare(qc)
            tw.wt = tw.wt.clone()
            tws.append(qc)
        x = torch.randn(max(16, args.n), k, device="cuda").to(torch.float16)
        if args.fp4:
            qs = []
            for c in range(copies):
                qc = QLinear(q.fmt, q.m, q.k, q.packed, q.scales, q.codes, q.row_scale, q.w)
                G.prepare_fp4(qc)
                qs.append(qc)
            out4 = torch.empty(16, m, dtype=torch.bfloat16, device="cuda")
            sks = [qs[0].kernel4.splitk] if args.splitk == "auto" else [int(s_) for s_ in args.splitk.split(",")]
            act = G.quantize_act_fp4(x, args.n, qs[0].kernel4.kp)
            for sk in sks:
                for qc in qs:
                    qc.kernel4.splitk = sk
                for mode in ("gemm", "quant+gemm"):
                    a = act if mode == "gemm" else None
                    for i in range(3):
                        G.linear_fp4(qs[i % copies], x, args.n, out=out4, act=a)
                    torch.cuda.synchronize()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for i in range(args.iters):
                        G.linear_fp4(qs[i % copies], x, args.n, out=out4, act=a)
                    e1.record()
                    torch.cuda.synchronize()
                    us = e0.elapsed_time(e1) * 1e3 / args.iters
                    print(json.dumps({"shape": name, "m": m, "k": k, "n": args.n, "path": "fp4 " + mode, "splitk": sk,
                                      "us": round(us, 2), "GBs": round(bytes_w / us / 1e3, 1)}))
            vlib.check_err_word()
            continue
        out = torch.empty(max(16, args.n), m, dtype=torch.bfloat16, device="cuda")
        sks = [tws[0].kernel.splitk] if args.splitk == "auto" else [int(s) for s in args.splitk.split(",")]
        for sk in sks:
            for qc in tws:
                qc.kernel.splitk = sk
            for i in range(3):
                G.linear(tws[i % copies], x, args.n, out=out)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(args.iters):
                G.linear(tws[i % copies], x, args.n, out=out)
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / args.iters
            print(json.dumps({"shape": name, "m": m, "k": k, "n": args.n, "splitk": sk, "us": round(us, 2),
                              "GBs": round(bytes_w / us / 1e3, 1)}))
        vlib.check_err_word()


if __name__ == "__main__":
    main()

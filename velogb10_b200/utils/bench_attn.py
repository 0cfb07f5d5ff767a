"""Decode attention micro-benchmark: the tensor-core split kernel against the CUDA-core one on one layer's worth of
KV cache (27B shape by default: 24 query / 4 KV heads, head_dim 256), CUDA-event timed, reported as achieved bytes/s
over the keys and values a step must read.

  python -m velogb10_b200.utils.bench_attn --ctx 4096,32768 --batch 1
"""
from __future__ import annotations

import argparse
import json

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ctx", default="2048,8192,32768")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--nh", type=int, default=24)
    ap.add_argument("--nkv", type=int, default=4)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--only", default="", help="tc | simt")
    args = ap.parse_args()
    from ..ops import kernels as K, lib
    dev = torch.device("cuda")
    hd, nh, nkv, n = 256, args.nh, args.nkv, args.batch
    for ctx in [int(c) for c in args.ctx.split(",")]:
        max_seq = ctx + 8
        # several cache copies so that consecutive iterations do not find the keys in L2
        copies = max(2, int(400e6 // (n * nkv * max_seq * hd * 4)) + 1)
        kcs = [torch.randn(n, nkv, max_seq, hd, device=dev).to(torch.bfloat16) for _ in range(copies)]
        vcs = [torch.randn(n, nkv, max_seq, hd, device=dev).to(torch.bfloat16) for _ in range(copies)]
        q = torch.randn(16, nh * hd, device=dev).to(torch.bfloat16)
        lens = torch.zeros(16, dtype=torch.int32, device=dev)
        lens[:n] = ctx
        slots = torch.arange(16, dtype=torch.int32, device=dev) % n
        part = torch.zeros(K.attn_scratch_floats(16, nh, hd, 32), device=dev)
        out = torch.zeros(16, nh * hd, dtype=torch.float16, device=dev)
        kv_bytes = 2 * n * nkv * ctx * hd * 2
        for name, fn in (("tc", K.attn_decode_tc), ("simt", K.attn_decode)):
            if args.only and args.only != name:
                continue
            for i in range(3):
                fn(q, kcs[i % copies], vcs[i % copies], lens, slots, part, out, n, nh, nkv, hd)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(args.iters):
                fn(q, kcs[i % copies], vcs[i % copies], lens, slots, part, out, n, nh, nkv, hd)
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / args.iters
            print(json.dumps({"kernel": name, "ctx": ctx, "batch": n, "us_split_plus_merge": round(us, 2),
                              "kv_GBs": round(kv_bytes / us / 1e3, 1)}))
        lib.check_err_word()


if __name__ == "__main__":
    main()

"""GatedDeltaNet prefill micro-benchmark on one layer's shapes (27B: 16 key / 48 value heads of 128 x 128): the
chunked tensor-core form against the exact recurrence kernel, CUDA-event timed, with the relative difference of the
outputs and of the final state.

  python -m velogb10_b200.utils.bench_gdn --tokens 2048,4096
"""
from __future__ import annotations

import argparse
import json

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", default="2048,4096")
    ap.add_argument("--nk", type=int, default=16)
    ap.add_argument("--nv", type=int, default=48)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--only", default="", help="chunked | exact")
    args = ap.parse_args()
    from ..ops import kernels as K, lib
    dev = "cuda"
    nk, nv, kd, vd = args.nk, args.nv, 128, 128
    key_dim, value_dim = nk * kd, nv * vd
    conv_dim = 2 * key_dim + value_dim
    ldp = (conv_dim + value_dim + 2 * nv + 7) // 8 * 8
    off = (conv_dim, conv_dim + value_dim, conv_dim + value_dim + nv)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    for T in [int(t) for t in args.tokens.split(",")]:
        torch.manual_seed(T)
        qkv = torch.randn(T, conv_dim, device=dev)
        proj = torch.randn(T, ldp, device=dev).to(torch.bfloat16)
        A_log, dt_bias = torch.randn(nv, device=dev) * 0.5, torch.randn(nv, device=dev) * 0.5
        norm_w = torch.rand(vd, device=dev) + 0.5
        S0 = torch.randn(2, nv, kd, vd, device=dev) * 0.1
        in_slot, out_slot = i32([0] * T), i32([-1] * (T - 1) + [1])
        work = torch.zeros(K.gdn_chunk_work_bytes(T, nv) + 1024, dtype=torch.uint8, device=dev)
        work = work[(-work.data_ptr()) % 1024:]
        o_raw = torch.zeros(T * value_dim, device=dev)
        outs, states, res = {}, {}, {}

        def chunked(S, o):
            K.gdn_chunk_prefill(qkv, proj, *off, S, A_log, dt_bias, norm_w, 0, T, in_slot, out_slot, o, nk, nv, kd, vd, 1e-6, work, o_raw)

        def exact(S, o):
            K.gdn_prefill(qkv, proj, *off, S, A_log, dt_bias, norm_w, 0, T, in_slot, out_slot, o, nk, nv, kd, vd, 1e-6,
                          o_scratch=o_raw, split=0)

        for name, fn in (("chunked", chunked), ("exact", exact)):
            if args.only and args.only != name:
                continue
            S = S0.clone()
            o = torch.zeros(T, value_dim, dtype=torch.float16, device=dev)
            fn(S, o)
            torch.cuda.synchronize()
            outs[name], states[name] = o.clone(), S.clone()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.iters):
                fn(S, o)
            e1.record()
            torch.cuda.synchronize()
            res[name] = e0.elapsed_time(e1) * 1e3 / args.iters
        lib.check_err_word()
        row = {"tokens": T, "nv": nv, "us": {k: round(v, 1) for k, v in res.items()}}
        if len(outs) == 2:
            rel = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm()).item()
            row["rel_out"] = rel(outs["chunked"], outs["exact"])
            row["rel_state"] = rel(states["chunked"][1], states["exact"][1])
        print(json.dumps(row))


if __name__ == "__main__":
    main()

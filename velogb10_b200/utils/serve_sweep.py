"""Continuous-batching + MTP speculative-verify sweep through the serving scheduler (no HTTP): R concurrent requests
with prompt lengths uniform in [512, 8192] and a fixed output length, greedy, for draft widths 0 (speculation off) and
1 / 2 / 4 forced on a random-weight draft head, followed by a second wave whose prompts extend the first wave's (the
prefix-cache hit path). Reports per cell: aggregate generated tok/s, decode-step latency percentiles (the verify-step
latency when speculating), prefill tokens computed vs reused, and whether the speculative output is bit-identical to
the non-speculative one. A width-N verify equals N decodes bit for bit while both run on the same GEMM path (steps of
at most 16 columns take the FP4-series GEMM, wider steps the f16-activation tensor-core GEMM): cells whose plain decode
step is wider than 16 lanes while the speculative forest verifies 16 columns at a time are marked
``mixed_gemm_paths`` and their comparison is informational (near-tie arg-max flips between two roundings).

  python -m velogb10_b200.utils.serve_sweep --model 27b --requests 4,8,16 --widths 0,1,2,4 --out-len 256
  python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \\
      -m velogb10_b200.utils.serve_sweep --tp --model 27b --requests 4,16,32

With ``--tp`` every rank runs the same deterministic schedule over its tensor-parallel shard (rank 0 prints).
With a random draft head nothing is accepted, so the speculative cells measure the cost side of speculation (draft
chain + wider verify); acceptance is a property of trained weights (reference: src/gpu.rs:6035-6213 ``--bench-mtp``).
"""
from __future__ import annotations

import argparse
import json
import os
import time

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="27b")
    ap.add_argument("--layers", type=int, default=0, help="keep only the first N layers (0 = full depth)")
    ap.add_argument("--requests", default="4,8,16")
    ap.add_argument("--widths", default="0,1,2,4")
    ap.add_argument("--out-len", type=int, default=256)
    ap.add_argument("--min-prompt", type=int, default=512)
    ap.add_argument("--max-prompt", type=int, default=8192)
    ap.add_argument("--seed", type=int, default=2)
    ap.add_argument("--tp", action="store_true")
    args = ap.parse_args()

    from ..checkpoint.synthetic import SyntheticSource
    from ..config import preset
    from ..engine.mtp import MtpPolicy
    from ..engine.sampling import SamplingParams
    from ..engine.scheduler import Request, Scheduler
    from ..models.runtime import GpuModel
    from ..models.weights import ModelBuilder
    from ..ops import lib as vlib

    rank, world, comm = 0, 1, None
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    if args.tp:
        import torch.distributed as dist
        from ..parallel.comm import TpComm
        rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
        dist.init_process_group("nccl", device_id=dev)
        comm = TpComm(rank, world, dev)
    cfg = preset(args.model, mtp=True)
    if args.layers and args.layers < cfg.num_layers:
        cfg.num_layers = args.layers
        cfg.layer_types = cfg.layer_types[:args.layers]
    reqs = [int(x) for x in args.requests.split(",")]
    widths = [int(x) for x in args.widths.split(",")]
    max_batch = max(reqs)
    max_seq = args.max_prompt + 2 * args.out_len + 64
    w = ModelBuilder(cfg, SyntheticSource(cfg, 0, str(dev)), recipe="all", device=str(dev), tp_rank=rank, tp_world=world).build()
    gm = GpuModel(w, device=str(dev), max_cols=max(16, max_batch), comm=comm)
    g = torch.Generator().manual_seed(args.seed)

    def prompts(n):
        lens = torch.randint(args.min_prompt, args.max_prompt + 1, (n,), generator=g).tolist()
        return [torch.randint(0, cfg.vocab_size - 2, (L,), generator=g).tolist() for L in lens]

    def run(prs, width, out_len, sched=None):
        pol = MtpPolicy("on", depth=width + 1, has_head=True) if width > 0 else MtpPolicy("off", has_head=True)
        sch = sched or Scheduler(gm, max_batch, max_seq, eos_ids=[], policy=pol, mtp_lanes=width > 0)
        sch.policy = pol
        outs = [[] for _ in prs]
        for i, p in enumerate(prs):
            sch.submit(Request(p, out_len, SamplingParams(temperature=0.0), on_token=outs[i].append))
        torch.cuda.synchronize(dev)
        t0 = time.time()
        sch.run_until_idle()
        torch.cuda.synchronize(dev)
        dt = time.time() - t0
        vlib.check_err_word(dev)
        return outs, sch, dt

    rows = []
    for R in reqs:
        prs = prompts(R)
        base = None
        for wd in widths:
            outs, sch, dt = run(prs, wd, args.out_len)
            if wd == 0 or base is None:
                base = outs if wd == 0 else base
            gen = sum(len(o) for o in outs)
            row = {"requests": R, "draft_width": wd, "prompt_tokens": sum(len(p) for p in prs), "generated": gen,
                   "wall_s": round(dt, 3), "agg_tok_s": round(gen / dt, 1),
                   "prefill_tokens_computed": sch.stats["prefill_tokens"], "step_latency_ms": {k: round(v, 3) for k, v in sch.latency_percentiles().items()},
                   "decode_steps": sch.stats["decode_steps"], "mtp_steps": sch.stats["mtp_steps"],
                   "forest_steps": sch.stats["forest_steps"], "graph_steps": sch.stats.get("graph_steps", 0),
                   "bit_identical_to_plain_greedy": (outs == base) if (wd > 0 and base is not None) else None,
                   "mixed_gemm_paths": bool(wd > 0 and R > 16)}
            if wd == 0:
                # prefix-cache hit path: every request again, extended by its own first 32 generated tokens
                t_pref0 = sch.stats["prefill_tokens"]
                ext = [p + o[:32] for p, o in zip(prs, outs)]
                outs2, sch, dt2 = run(ext, 0, 32, sched=sch)
                row["prefix_hit_wave"] = {"wall_s": round(dt2, 3), "prefill_tokens_computed": sch.stats["prefill_tokens"] - t_pref0,
                                          "prefill_tokens_if_cold": sum(len(p) for p in ext),
                                          "live_hits": sch.stats["prefix_live"], "ckpt_hits": sch.stats["prefix_ckpt"]}
            rows.append(row)
            if rank == 0:
                print(json.dumps(row), flush=True)
    if rank == 0:
        print(json.dumps({"sweep": "continuous batching + MTP verify", "model": cfg.name, "layers": cfg.num_layers, "tp": world,
                          "out_len": args.out_len, "rows": len(rows)}))
    if args.tp:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()

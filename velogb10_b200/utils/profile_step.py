"""Runs a few eager steps of a (possibly depth-reduced) preset model between cudaProfilerStart/Stop, so a
profiler attached with ``--profile-from-start off`` sees only those steps.

  python -m velogb10_b200.utils.profile_step --model 27b --layers 8 --mode decode --steps 1
  ncu --metrics gpu__time_duration.sum --clock-control none --profile-from-start off --csv \
      --log-file launches.csv python -m velogb10_b200.utils.profile_step --model 27b --layers 8

Without a profiler it prints CUDA-event timings of the same steps. ``--layers`` keeps the per-layer
shapes and the 3:1 layer pattern of the preset, so per-kernel times are those of the full model.
"""
from __future__ import annotations

import argparse
import json

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="27b")
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--mode", default="decode", choices=["decode", "verify", "prefill", "spec"],
                    help="spec: one sampled decode (device penalties / top-k / nucleus draw), one draft-head step and one "
                         "stochastic chain verify with the device accept kernel: the kernels of the speculative serving path")
    ap.add_argument("--steps", type=int, default=1)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--width", type=int, default=4)
    ap.add_argument("--ctx", type=int, default=512)
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--recipe", default="all")
    ap.add_argument("--tp", action="store_true", help="tensor parallel over the ranks of a torchrun job (rank 0 prints)")
    ap.add_argument("--kernel-times", action="store_true",
                    help="print the in-stream duration of every kernel of the timed steps (activity tracing, no "
                         "replay: warm caches and real overlap, unlike a per-kernel profiler capture)")
    args = ap.parse_args()

    from ..config import preset
    from ..engine.llm import LLM

    from ..ops import lib as vlib

    import os
    rank, world, comm = 0, 1, None
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    if args.tp:
        import torch.distributed as dist
        from ..parallel.comm import TpComm
        rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
        dist.init_process_group("nccl", device_id=dev)
        comm = TpComm(rank, world, dev)
    cfg = preset(args.model, mtp=args.mode == "spec")
    if args.layers and args.layers < cfg.num_layers:
        cfg.num_layers = args.layers
        cfg.layer_types = cfg.layer_types[:args.layers]
    llm = LLM.synthetic(cfg, recipe=args.recipe, device=str(dev), max_batch=max(4, args.batch),
                        max_seq=max(args.ctx, args.prompt) + 64, tp_rank=rank, tp_world=world, comm=comm)
    gm = llm.model
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, cfg.vocab_size, (max(args.ctx, args.prompt),), generator=g).tolist()
    for s in range(args.batch):
        gm.prefill(s, toks[:args.ctx], 0, want_hidden=False)

    def step(i):
        if args.mode == "decode":
            gm.decode([1 + i] * args.batch, [args.ctx + i] * args.batch, list(range(args.batch)))
        elif args.mode == "verify":
            gm.verify(0, list(range(1, 1 + args.width)), args.ctx, ckpt_base=args.batch)
        elif args.mode == "spec":
            from ..engine.sampling import SamplingParams
            sp = SamplingParams(0.8, 0.9, 20, 1.1, 0.5, 0.1, seed=1)
            logits, hidden = gm.decode([1 + i], [args.ctx], [0])
            gm.sampler.pick(logits.float(), [sp], [[1, 2, 3, 2]], [7 + i])                     # sampled decode
            h = hidden[:1].clone()
            gm.mtp_forward(0, [2 + i], h, [args.ctx - 1])                                       # draft-head step
            drafts = list(range(2, 1 + args.width))
            lv, _ = gm.verify(0, [1 + i] + drafts, args.ctx, ckpt_base=args.batch)            # chain verify
            gm.sampler.chain_accept(lv.float(), sp, [1, 2, 3, 2], drafts, 11 + i)               # accept / resample
        else:
            gm.prefill(1 % max(args.batch, 2), toks[:args.prompt], 0, want_hidden=False)

    step(0)
    torch.cuda.synchronize()
    n_launch = vlib.count_launches(lambda: step(1))
    torch.cuda.synchronize()
    if args.kernel_times:
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for i in range(args.steps):
                step(2 + i)
            torch.cuda.synchronize()
        rows = []
        for ev in prof.key_averages():
            us = getattr(ev, "device_time_total", None)
            if us is None:
                us = getattr(ev, "cuda_time_total", 0.0)
            if us > 0:
                rows.append((us / args.steps, ev.count // args.steps, ev.key))
        total = sum(r[0] for r in rows)
        if rank == 0:
            for us, cnt, name in sorted(rows, reverse=True)[:24]:
                print(f"{us:10.1f} us {100 * us / total:5.1f}% x{cnt:<4d} {name[:110]}")
            print(f"{total:10.1f} us total kernel time per step")
        if args.tp:
            dist.destroy_process_group()
        return
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.profiler.start()
    e0.record()
    for i in range(args.steps):
        step(2 + i)
    e1.record()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    vlib.check_err_word()
    if rank == 0:
        print(json.dumps({"mode": args.mode, "layers": cfg.num_layers, "steps": args.steps,
                          "ms_per_step_eager": e0.elapsed_time(e1) / args.steps, "launches_per_step": n_launch}))
    if args.tp:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

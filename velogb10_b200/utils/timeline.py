"""Device timeline of one CUDA-graph decode step: which kernel (and which phase of it) is running when.

Needs a library built with the timeline stamps compiled in (``VELO_TRACE=1 python -m velogb10_b200.ops.build``):
``trace()`` in ``csrc/common.cuh`` then appends (``%globaltimer``, event code, block) records to a buffer. Prints
the records of block 0 of every kernel in time order (microseconds from the first record).

  VELO_TRACE=1 python -m velogb10_b200.ops.build
  VELO_TRACE=1 python -m velogb10_b200.utils.timeline --model 27b --layers 8
  VELO_TRACE=1 torchrun --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 -m velogb10_b200.utils.timeline --tp

Event codes: kernel * 16 + event; kernels 1 = residual/RMSNorm/quantise, 2 = quantiser (SwiGLU or plain), 4 = FP4
GEMM, 5 = conv, 6 = GDN recurrence; events 0 = entry, 1 = dependency wait returned, 2 = end, 3 = first operands
landed, 4 = accumulator complete, 5 = prologue done, 6 = all-reduce values published, 8 = accumulators read out of
TMEM, 9 / 10 = split-K partials visible across the cluster / reduced, 11 = outputs stored.
"""
from __future__ import annotations

import argparse
import ctypes
import os

import torch

KERNELS = {1: "norm_q", 2: "quant", 4: "gemm", 5: "conv", 6: "gdn"}
EVENTS = {0: "entry", 1: "waited", 2: "end", 3: "first_full", 4: "acc_full", 5: "prologue_done", 6: "ar_published",
          7: "ar_flags_seen", 8: "acc_in_registers", 9: "splitk_partials_visible", 10: "splitk_reduced", 11: "outputs_stored"}
# events whose meaning differs per kernel, and the ones printed from whichever block records them (the GDN row
# quantisation runs in the last head to finish, not in block 0)
PER_KERNEL = {1 * 16 + 3: "sum_of_squares_reduced", 1 * 16 + 4: "row_max_reduced", 2 * 16 + 3: "cta_max_reduced",
              2 * 16 + 4: "cluster_max_known", 6 * 16 + 3: "head_outputs_stored", 6 * 16 + 4: "row_quantise_begins",
              6 * 16 + 5: "row_quantise_done"}
ANY_BLOCK = {6 * 16 + 4, 6 * 16 + 5}
SETTERS = ("vg_trace_set_act_quant", "vg_trace_set_gdn", "vg_trace_set_gemm_fp4")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="27b")
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=512)
    ap.add_argument("--tp", action="store_true", help="tensor parallel over the ranks of the torchrun job (prints rank 0)")
    ap.add_argument("--until-us", type=float, default=400.0)
    args = ap.parse_args()

    from ..config import preset
    from ..engine.llm import LLM
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
    cfg = preset(args.model, mtp=False)
    if args.layers and args.layers < cfg.num_layers:
        cfg.num_layers, cfg.layer_types = args.layers, cfg.layer_types[:args.layers]
    llm = LLM.synthetic(cfg, recipe="all", device=str(dev), max_batch=4, max_seq=args.ctx + 128, tp_rank=rank,
                        tp_world=world, comm=comm)
    gm = llm.model
    toks = torch.randint(0, cfg.vocab_size, (args.ctx,), generator=torch.Generator().manual_seed(1)).tolist()
    gm.prefill(0, toks, 0, want_hidden=False)
    gm.capture_decode(1)
    for i in range(3):
        gm.replay_decode([5], [args.ctx + i], [0])
    torch.cuda.synchronize()
    cap = 1 << 16
    buf = torch.zeros(1 + 2 * cap, dtype=torch.int64, device=dev)
    L = vlib.lib()
    for fn in SETTERS:
        rc = getattr(L, fn)(ctypes.c_void_p(buf.data_ptr()), ctypes.c_uint(cap))
        if rc != 0:
            raise SystemExit("this library was built without the timeline stamps (VELO_TRACE=1)")
    torch.cuda.synchronize()
    if args.tp:
        dist.barrier()
    gm.replay_decode([5], [args.ctx + 3], [0])
    torch.cuda.synchronize()
    for fn in SETTERS:
        getattr(L, fn)(ctypes.c_void_p(0), ctypes.c_uint(0))
    if rank == 0:
        b = buf.cpu()
        n = int(b[0].item()) & 0xffffffff
        rec = sorted((int(b[1 + 2 * i]), int(b[2 + 2 * i])) for i in range(min(n, cap)))
        t0 = rec[0][0] if rec else 0
        for t, w in rec:
            code, bx, bz = w & 0xffff, (w >> 32) & 0xffffffff, (w >> 16) & 0xffff
            us = (t - t0) / 1000.0
            if us > args.until_us:
                break
            name = PER_KERNEL.get(code, EVENTS.get(code & 15, code & 15))
            if (bx == 0 and bz == 0) or code in ANY_BLOCK:
                print(f"{us:9.2f} {KERNELS.get(code >> 4, code >> 4):7} {name}" + (f" (block {bx})" if bx else ""))
        print("records", n)
    if args.tp:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

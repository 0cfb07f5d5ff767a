"""Mixture-of-experts FFN on the GPU: router -> (per-pair decode path | sorted grouped prefill path) ->
slot-order combine -> expert-parallel reduction -> gated shared expert.

Counterpart of the reference's ``moe_batch`` (reference: src/gpu.rs:2199-2414): the decode / verify path
(<= 16 columns) runs one grouped-GEMM work item per (token, slot) pair, so every column is computed the same
way whatever the batch width; longer inputs are sorted by expert on the device and run through the grouped
tensor-core GEMM with 128-token tiles. Under expert parallelism each rank holds a contiguous band of
experts, computes only its pairs and the partial outputs are summed with the peer-memory all-reduce before
the replicated shared expert is added.
"""
from __future__ import annotations

import contextlib
import ctypes
import os

from typing import Dict

import torch

from ..ops import gemm as G
from ..ops import kernels as K
from ..ops import lib as _lib
from ..ops.lib import c_float, c_int, ptr, stream
from .weights import MoeW

DECODE_MAX = 16


class MoeBuffers:
    def __init__(self, cfg, M: MoeW, cap: int, dev):
        E, topk, I, h = cfg.num_experts, cfg.num_experts_per_tok, cfg.moe_intermediate_size, cfg.hidden_size
        P = cap * topk
        i32 = lambda *s: torch.zeros(s, dtype=torch.int32, device=dev)
        self.cap, self.P = cap, P
        self.logits = torch.zeros((cap, E), dtype=torch.float32, device=dev)
        self.ids, self.wts = i32(P), torch.zeros(P, dtype=torch.float32, device=dev)
        ng = max(P, M.n_local)
        self.g_exp, self.g_off, self.g_cnt = i32(ng), i32(ng), i32(ng)
        rows = max(P, 16) + 128
        self.gu = torch.zeros((rows, 2 * I), dtype=torch.bfloat16, device=dev)
        self.a16 = torch.zeros((rows, I), dtype=torch.float16, device=dev)
        self.y = torch.zeros((rows, h), dtype=torch.bfloat16, device=dev)
        self.gate_logit = torch.zeros((max(cap, 16), 1), dtype=torch.float32, device=dev)
        self.shared = torch.zeros((max(cap, 16), h), dtype=torch.bfloat16, device=dev)
        if cap > DECODE_MAX:
            self.max_items = (P + 127) // 128 + M.n_local
            self.cnt, self.cursor = i32(M.n_local), i32(M.n_local)
            self.tilemap, self.n_items, self.total = i32(self.max_items, 2), i32(1), i32(1)
            self.perm, self.inv = i32(P), i32(P)
            self.xperm = torch.zeros((rows, h), dtype=torch.float16, device=dev)


def _buffers(model, ws, M: MoeW) -> MoeBuffers:
    cache: Dict = model.__dict__.setdefault("_moe_bufs", {})
    key = (id(ws), M.n_local)
    b = cache.get(key)
    if b is None:
        b = MoeBuffers(model.cfg, M, ws.cap, model.dev)
        cache[key] = b
    return b


def _prep_experts(q, fp4: bool):
    """Tile-major layouts of a stacked expert tensor (each expert's rows are a multiple of 128): the 16-bit-MMA
    tiles for sorted prefill and, for NVFP4 experts, the FP4 tiles for the per-pair decode path."""
    if fp4 and q.fmt == "nvfp4" and getattr(q, "kernel4", None) is None and q.packed is not None:
        G.prepare_fp4(q, splitk=1)
    tw = G.prepare(q, keep_canonical=False, splitk=1)
    return tw


def _grouped(tw, m_per_expert, x16, out, bn, max_items, g_exp, g_off, g_cnt, tilemap, n_items, x_div, dev):
    rc = _lib.lib().vg_gemm_tc_grouped(ptr(tw.wt), ptr(tw.row_scale), ptr(x16), c_int(x16.shape[0]), c_int(x16.stride(0)),
                                       ptr(out), c_int(0), c_int(m_per_expert), c_int(tw.k), c_int(out.stride(0)),
                                       c_int(tw.fmt), c_int(bn), c_int(max_items), ptr(g_exp), ptr(g_off), ptr(g_cnt),
                                       ptr(tilemap), ptr(n_items), c_int(x_div), ptr(_lib.err_word(dev)), stream())
    _lib.check(rc, "vg_gemm_tc_grouped")


def _small_linear(q, x16, n: int, out):
    """Router / shared-gate logits (fp32): the CUDA-core GEMV at decode widths, the tensor-core GEMM over f16
    tiles of the same weights for prefill widths (the GEMV walks the columns one by one)."""
    if n > 16 and getattr(q, "kernel", None) is not None:
        G.linear(q, x16, n, out=out, out_f32=True)
    else:
        G.linear_simt(q, x16, n, out=out, out_f32=True)


def moe_forward(model, ws, M: MoeW, n: int, act=None):
    """Reads ws.xn16[:n] (normed hidden, f16); writes the FFN output into ws.delta[:n] (bf16)."""
    cfg = model.cfg
    L = _lib.lib()
    E, topk, I, h = cfg.num_experts, cfg.num_experts_per_tok, cfg.moe_intermediate_size, cfg.hidden_size
    b = _buffers(model, ws, M)
    gu_w, dn_w = _prep_experts(M.gate_up, model.use_fp4), _prep_experts(M.down, model.use_fp4)
    # The shared expert does not depend on the routing: at decode widths it runs on a second stream beside the
    # routed experts (a fork / join that CUDA-graph capture records as two branches) and meets them at the combine.
    shared = gate = joined = None
    if M.shared is not None:
        fork = n <= 16 and model.moe_side_stream is not None
        if fork:
            main = torch.cuda.current_stream()
            model.moe_fork_event.record(main)
            model.moe_side_stream.wait_event(model.moe_fork_event)
            ctx = torch.cuda.stream(model.moe_side_stream)
        else:
            ctx = contextlib.nullcontext()
        with ctx:
            model._mlp(ws, M.shared, n, b.shared, reduce=False, act=act, buf_tag="shared" if fork else "")
            shared = b.shared
            if M.shared_gate is not None:
                _small_linear(M.shared_gate, ws.xn16, n, b.gate_logit)
                gate = b.gate_logit
            if fork:
                joined = model.moe_join_event
                joined.record(model.moe_side_stream)
    _small_linear(M.router, ws.xn16, n, b.logits)
    hook = getattr(model, "router_logits_hook", None)
    if hook is not None:
        # test / analysis hook: sees (and may overwrite) the fp32 router logits [n, E] before the top-k selection,
        # e.g. to replay another run's routing so that two runs differ only in how the expert outputs are summed
        hook(b.logits, n)
    P = n * topk
    decode = ws.cap <= DECODE_MAX
    rc = L.vg_moe_router(ptr(b.logits), c_int(n), c_int(E), c_int(topk), c_int(1 if cfg.router_sigmoid else 0),
                         ptr(M.expert_bias if cfg.router_expert_bias else None), c_int(1 if cfg.route_norm else 0),
                         c_float(cfg.router_scaling), c_int(M.e_base), c_int(M.n_local), ptr(b.ids), ptr(b.wts),
                         ptr(b.g_exp if decode else None), ptr(b.g_off if decode else None),
                         ptr(b.g_cnt if decode else None), stream())
    _lib.check(rc, "vg_moe_router")
    fp4 = (decode and act is not None and getattr(M.gate_up, "kernel4", None) is not None
           and getattr(M.down, "kernel4", None) is not None and (2 * I) % 128 == 0 and h % 128 == 0 and I % 8 == 0)
    if fp4:
        # per-pair FP4 path: the token's quantised series feeds every selected expert's gate_up; SwiGLU emits one
        # quantised row per pair (own buffers: the shared expert quantises on the other stream) for the down GEMM
        G.linear_fp4_grouped(M.gate_up, act, b.gu, b.g_exp, b.g_off, P, topk, 2 * I)
        act_p = G.swiglu_fp4(b.gu, P, I, bufs=G.fp4_buffers(model.dev, ((I + 255) // 256) * 256, rows=b.P, tag="moe"))
        G.linear_fp4_grouped(M.down, act_p, b.y, b.g_exp, b.g_off, P, 1, h)
    elif decode:
        _grouped(gu_w, 2 * I, ws.xn16, b.gu, 16, P, b.g_exp, b.g_off, b.g_cnt, None, None, topk, model.dev)
        K.swiglu(b.gu, b.a16, P, I)
        _grouped(dn_w, h, b.a16, b.y, 16, P, b.g_exp, b.g_off, b.g_cnt, None, None, 1, model.dev)
    if decode:
        inv = None
        # non-resident pairs were skipped by the GEMM: make the combine skip them too
        if M.n_local < E:
            inv = b.g_exp_inv = getattr(b, "g_exp_inv", None)
            if inv is None:
                inv = b.g_exp_inv = torch.zeros(b.P, dtype=torch.int32, device=model.dev)
            torch.where(b.g_exp[:P] >= 0, b.g_off[:P], torch.full_like(b.g_off[:P], -1), out=inv[:P])
    else:
        rc = L.vg_moe_sort(ptr(b.ids), c_int(P), c_int(M.e_base), c_int(M.n_local), c_int(128), ptr(b.cnt), ptr(b.cursor),
                           ptr(b.g_exp), ptr(b.g_off), ptr(b.g_cnt), ptr(b.tilemap), ptr(b.n_items), ptr(b.perm),
                           ptr(b.inv), ptr(b.total), stream())
        _lib.check(rc, "vg_moe_sort", 5)
        rc = L.vg_moe_gather(ptr(ws.xn16), c_int(ws.xn16.stride(0)), ptr(b.perm), ptr(b.total), c_int(P), c_int(topk),
                             c_int(h), ptr(b.xperm), stream())
        _lib.check(rc, "vg_moe_gather")
        items = (P + 127) // 128 + M.n_local
        _grouped(gu_w, 2 * I, b.xperm, b.gu, 128, items, b.g_exp, b.g_off, b.g_cnt, b.tilemap, b.n_items, 1, model.dev)
        K.swiglu(b.gu, b.a16, P, I)
        _grouped(dn_w, h, b.a16, b.y, 128, items, b.g_exp, b.g_off, b.g_cnt, b.tilemap, b.n_items, 1, model.dev)
        inv = b.inv
    if joined is not None:
        torch.cuda.current_stream().wait_event(joined)
    ep = model.comm is not None and model.comm.world > 1 and M.n_local < E
    comm = model.comm
    if ep and decode and model.use_fp4 and model.split_allreduce and model.fuse_allreduce and not comm.use_nccl \
            and h % 16 == 0 and n * h * 8 <= comm.slot_bytes and os.environ.get("VELO_NO_MOE_PUSH", "0") != "1":
        # combine fused with the expert-parallel all-reduce: the partial rows go straight into every rank's receive
        # slots and the next residual-add / RMSNorm kernel sums them (rank 0 contributes the replicated shared expert)
        # a sharded shared expert contributes a partial on every rank; a replicated one is added by rank 0 only
        first = comm.rank == 0 or getattr(M.shared, "partial", False)
        rc = L.vg_moe_combine_push(ptr(b.y), c_int(b.y.stride(0)), ptr(inv), ptr(b.wts), c_int(n), c_int(topk),
                                   ptr(shared if first else None), ptr(gate if first else None), c_int(h),
                                   ctypes.byref(comm.ctx), stream())
        _lib.check(rc, "vg_moe_combine_push")
        model._pending_ar = 1
        return
    sh_partial = ep and shared is not None and getattr(M.shared, "partial", False)
    with_shared = (not ep) or sh_partial
    rc = L.vg_moe_combine(ptr(b.y), c_int(b.y.stride(0)), ptr(inv), ptr(b.wts), c_int(n), c_int(topk),
                          ptr(shared if with_shared else None), ptr(gate if with_shared else None), ptr(ws.delta), c_int(h),
                          stream())
    _lib.check(rc, "vg_moe_combine")
    if ep:
        comm.all_reduce_rows(ws.delta, n)
        if shared is not None and not sh_partial:
            rc = L.vg_moe_add_shared(ptr(ws.delta), ptr(shared), ptr(gate), c_int(n), c_int(h), stream())
            _lib.check(rc, "vg_moe_add_shared")

"""Tensor-parallel communicator over NVLink peer memory.

``TpComm`` allocates this rank's symmetric arena, exchanges CUDA IPC handles through ``torch.distributed``
(the process group is only used for this bootstrap, for barriers and as the measured baseline), maps every
peer's arena and drives the peer-memory kernels of ``csrc/comm.cu``: one-shot / two-shot all-reduce with
rank-order fp32 sums, small all-gather, and the vocabulary-parallel arg-max merge. ``use_nccl=True``
switches every collective to the library implementation (the comparison baseline, never the default).
It replaces the reference's two-node RDMA link (reference: src/net.rs:151-267, src/tp.rs:116-188).
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import lib as _lib
from ..ops.lib import c_int, c_ll, ptr, stream

FLAGS_BYTES = 4 * 8 * 64 * 128
CTRL_BYTES = 256


class VgCommCtx(ctypes.Structure):
    _fields_ = [("rank", ctypes.c_int), ("world", ctypes.c_int), ("data", ctypes.c_void_p * 8),
                ("flags_off", ctypes.c_ulonglong), ("slots_off", ctypes.c_ulonglong), ("slot_bytes", ctypes.c_ulonglong),
                ("result_off", ctypes.c_ulonglong), ("result_bytes", ctypes.c_ulonglong),
                ("epoch", ctypes.c_void_p), ("done_ctr", ctypes.c_void_p), ("status", ctypes.c_void_p),
                ("timeout_ns", ctypes.c_ulonglong), ("agbuf_off", ctypes.c_ulonglong), ("agbuf_bytes", ctypes.c_ulonglong),
                ("agflags_off", ctypes.c_ulonglong), ("rsflags_off", ctypes.c_ulonglong),
                ("mc", ctypes.c_void_p), ("mm_off", ctypes.c_ulonglong), ("mm_slot_bytes", ctypes.c_ulonglong),
                ("mmflags_off", ctypes.c_ulonglong), ("mm_ctr", ctypes.c_void_p)]


RS_MAX_TILES = 4096                      # per-tile epoch words of the fused GEMM + reduce-scatter, per (set, rank)
AG_MAX_TILES = 256                       # per-tile epoch words of the fused all-gather + GEMM, per set
MM_SLOT_BYTES = 1 << 20                  # fp32 partial rows of one decode-width collective (16 rows x 16384 columns)
ARGMAX_MAX_COLS = 64                     # columns the arg-max merge buffers hold (csrc/api.h VG_ARGMAX_MAX_COLS)


class CommError(RuntimeError):
    pass


class TpComm:
    def __init__(self, rank: int, world: int, device: torch.device, max_elems: int = 4096 * 8192, use_nccl: bool = False,
                 timeout_s: float = 5.0, group=None, ag_bytes: int = 0):
        self.rank, self.world, self.dev = rank, world, torch.device(device)
        self.use_nccl = use_nccl
        self.group = group
        self.L = _lib.lib()
        seg = ((max_elems + world - 1) // world + 7) & ~7
        # a slot must hold a whole one-shot vector (<= 1 Mi elements) or one two-shot segment, in fp32
        self.slot_bytes = max(seg * 4, 4 << 20)
        self.result_bytes = ((seg * world * 2 + 255) // 256) * 256
        self.flags_off = CTRL_BYTES
        self.slots_off = self.flags_off + FLAGS_BYTES
        self.result_off = self.slots_off + 2 * 8 * self.slot_bytes
        self.rsflags_off = self.result_off + 2 * self.result_bytes
        self.agflags_off = self.rsflags_off + 2 * 8 * RS_MAX_TILES * 4
        self.agbuf_off = (self.agflags_off + 2 * AG_MAX_TILES * 4 + 1023) // 1024 * 1024
        self.agbuf_bytes = (ag_bytes + 1023) // 1024 * 1024      # two landing zones of the fused all-gather + GEMM
        self.mmflags_off = (self.agbuf_off + self.agbuf_bytes + 1023) // 1024 * 1024
        self.mm_off = self.mmflags_off + 4096          # flags: [2 sets][64 tiles][8 ranks] words
        self.total = self.mm_off + 2 * MM_SLOT_BYTES
        self.mc = 0                     # multicast (NVLS) address of the arena, 0 when it has none
        self.arena_kind = "cuda-ipc"
        self._symm = None
        self._symm_bufs = []
        with torch.cuda.device(self.dev):
            # Preferred substrate: a symmetric allocation with an NVLink-switch multicast binding (torch's symmetric
            # memory does the allocation and the handle exchange), which adds in-switch reductions to the peer
            # pointers. VELO_NO_MULTIMEM=1 keeps the plain CUDA-IPC arena (peer loads / stores only): required for
            # drills in which a rank may leave, since a dead rank must not hold memory bound to a multicast object.
            if os.environ.get("VELO_NO_MULTIMEM", "0") != "1" and not use_nccl:
                try:
                    self._alloc_symmetric(group)
                except Exception as e:  # noqa: BLE001 - any failure: the IPC arena serves every peer-pointer path
                    self.arena_note = f"symmetric memory unavailable ({type(e).__name__}: {str(e)[:120]})"
                    self._symm = None
            if self._symm is None:
                self._alloc_ipc(group)
        ctx = VgCommCtx()
        ctx.rank, ctx.world = rank, world
        for q in range(8):
            ctx.data[q] = self.peers[q] if q < world else None
        ctx.flags_off, ctx.slots_off, ctx.slot_bytes = self.flags_off, self.slots_off, self.slot_bytes
        ctx.result_off, ctx.result_bytes = self.result_off, self.result_bytes
        ctx.epoch, ctx.done_ctr, ctx.status = self.base, self.base + 4, self.base + 8
        ctx.timeout_ns = int(timeout_s * 1e9)
        ctx.rsflags_off = self.rsflags_off
        ctx.agbuf_off, ctx.agbuf_bytes, ctx.agflags_off = self.agbuf_off, self.agbuf_bytes, self.agflags_off
        ctx.mc = self.mc or None
        ctx.mm_off, ctx.mm_slot_bytes, ctx.mmflags_off = self.mm_off, MM_SLOT_BYTES, self.mmflags_off
        ctx.mm_ctr = self.base + 12
        self.ctx = ctx
        # decode-width all-reduce through the switch (multimem.ld_reduce) when the arena has a multicast address
        # (measured on 2 and on 4 GPUs the pair push is the faster of the two: one NVLink hop instead of flag + reduce
        # round trip, 198 vs 182 and 216 vs 206 tok/s; its cost grows with the number of ranks, the in-switch form's
        # does not)
        mm_min = int(os.environ.get("VELO_MULTIMEM_MIN_WORLD", "8"))
        self.use_mm = bool(self.mc) and world >= mm_min
        self._status_view = self._view(8, 1, torch.int32)
        self._pairs = torch.zeros(2 * ARGMAX_MAX_COLS, dtype=torch.float32, device=self.dev)
        self._gathered = torch.zeros(2 * ARGMAX_MAX_COLS * world, dtype=torch.float32, device=self.dev)
        self._out_tok = torch.zeros(ARGMAX_MAX_COLS, dtype=torch.int32, device=self.dev)
        self._val = torch.zeros(ARGMAX_MAX_COLS, dtype=torch.float32, device=self.dev)
        self._idx = torch.zeros(ARGMAX_MAX_COLS, dtype=torch.int32, device=self.dev)
        dist.barrier(group=group)

    def _alloc_ipc(self, group):
        base = ctypes.c_void_p()
        _lib.check(self.L.vg_comm_alloc(ctypes.byref(base), ctypes.c_ulonglong(self.total)), "vg_comm_alloc")
        self.base = base.value
        hb = self.L.vg_comm_handle_bytes()
        handle = (ctypes.c_ubyte * hb)()
        _lib.check(self.L.vg_comm_export(base, handle), "vg_comm_export")
        mine = bytes(handle)
        handles: List[Optional[bytes]] = [None] * self.world
        dist.all_gather_object(handles, mine, group=group)
        self.peers: List[int] = []
        for q in range(self.world):
            if q == self.rank:
                self.peers.append(self.base)
                continue
            p = ctypes.c_void_p()
            buf = (ctypes.c_ubyte * hb).from_buffer_copy(handles[q])
            _lib.check(self.L.vg_comm_import(buf, ctypes.byref(p)), "vg_comm_import")
            self.peers.append(p.value)

    def _alloc_symmetric(self, group):
        import torch.distributed._symmetric_memory as symm
        t = symm.empty(self.total, dtype=torch.uint8, device=self.dev)
        hdl = symm.rendezvous(t, group if group is not None else dist.group.WORLD)
        off = int(getattr(hdl, "offset", 0) or 0)
        peers = [int(p) + off for p in hdl.buffer_ptrs]
        if len(peers) != self.world or peers[self.rank] != t.data_ptr():
            raise RuntimeError("symmetric memory handle does not describe this allocation")
        t.zero_()
        torch.cuda.synchronize(self.dev)
        self._symm = (t, hdl)
        self.base, self.peers = t.data_ptr(), peers
        mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
        self.mc = mc + off if mc else 0
        self.arena_kind = "symmetric+multicast" if self.mc else "symmetric"

    def symmetric_buffer(self, nbytes: int):
        """A uint8 tensor in multicast-bound symmetric memory (collective: every rank calls it in the same order with the
        same size), or None when the arena has no multicast binding. Buffers obtained here can be reduced in place with
        ``all_reduce_multimem``."""
        if not self.mc:
            return None
        import torch.distributed._symmetric_memory as symm
        with torch.cuda.device(self.dev):
            t = symm.empty(nbytes, dtype=torch.uint8, device=self.dev)
            hdl = symm.rendezvous(t, self.group if self.group is not None else dist.group.WORLD)
            mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
            off = int(getattr(hdl, "offset", 0) or 0)
            if not mc:
                return None
            t.zero_()
            torch.cuda.synchronize(self.dev)
        self._symm_bufs.append((t.data_ptr(), nbytes, mc + off, t, hdl))
        dist.barrier(group=self.group)
        return t

    def multicast_address(self, t: torch.Tensor) -> int:
        """Multicast address of a tensor that lives inside a ``symmetric_buffer`` (0 if it does not)."""
        p = t.data_ptr()
        for base, nbytes, mc, _, _ in self._symm_bufs:
            if base <= p and p + t.numel() * t.element_size() <= base + nbytes:
                return mc + (p - base)
        return 0

    def all_reduce_multimem(self, t: torch.Tensor, n_rows: int) -> bool:
        """In-place sum over ranks of the first rows of a bf16 tensor inside a symmetric buffer, reduced inside the
        NVLink switch. Returns False (nothing done) when the tensor is not multicast-addressable."""
        mc = self.multicast_address(t)
        n = n_rows * t.shape[1]
        if not mc or t.dtype != torch.bfloat16 or not t.is_contiguous() or n % 8 or self.use_nccl:
            return False
        rc = self.L.vg_comm_allreduce_multimem(ctypes.byref(self.ctx), ctypes.c_void_p(mc), c_ll(n), stream())
        _lib.check(rc, "vg_comm_allreduce_multimem")
        return True

    def describe(self) -> dict:
        """How this communicator moves data (recorded next to benchmark numbers)."""
        return {"arena": self.arena_kind, "multicast": bool(self.mc), "note": getattr(self, "arena_note", ""),
                "decode_allreduce": "nccl" if self.use_nccl else
                ("in-switch multimem.ld_reduce of fp32 partials fused into GEMM epilogue + norm" if self.use_mm else
                 "(value, epoch) pair push to every rank fused into GEMM epilogue + norm"),
                "world": self.world}

    def _view(self, offset: int, n: int, dtype) -> torch.Tensor:
        """Torch view of a piece of this rank's arena."""
        class _Arr:
            pass
        a = _Arr()
        item = torch.tensor([], dtype=dtype).element_size()
        typestr = {torch.int32: "<i4", torch.float32: "<f4", torch.uint8: "|u1", torch.float16: "<f2"}[dtype]
        a.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (self.base + offset, False), "version": 2}
        return torch.as_tensor(a, device=self.dev)

    # ------------------------------------------------------------ collectives
    def all_reduce_rows(self, t: torch.Tensor, n_rows: int):
        """In-place sum over ranks of the first ``n_rows`` rows of a contiguous bf16/f32 ``[rows, h]`` tensor."""
        n = n_rows * t.shape[1]
        if n_rows > 64 and self._symm_bufs and self.all_reduce_multimem(t, n_rows):
            return
        if self.use_nccl:
            dist.all_reduce(t[:n_rows], group=self.group)
            return
        assert t.is_contiguous() and t.dtype in (torch.bfloat16, torch.float32)
        is32 = t.dtype == torch.float32
        rc = self.L.vg_comm_allreduce(ctypes.byref(self.ctx), ptr(t), c_int(1 if is32 else 0),
                                      ptr(None if is32 else t), ptr(t if is32 else None), c_ll(n), stream())
        _lib.check(rc, "vg_comm_allreduce")

    def rs_rows_for(self, n_rows: int, m: int) -> int:
        """Token rows per rank for the fused GEMM + reduce-scatter of an ``[n_rows, m]`` output (whole 128-token
        tiles), or 0 when the shape does not fit the arena."""
        rows = ((n_rows + self.world - 1) // self.world + 127) // 128 * 128
        tiles = (rows // 128) * ((m + 127) // 128)
        if m % 8:
            return 0
        if tiles > RS_MAX_TILES or rows * m * 4 > self.slot_bytes or rows * self.world * m * 2 > self.result_bytes:
            return 0
        return rows

    def gemm_rs_finish(self, out: torch.Tensor, n_rows: int, rs_rows: int):
        """Second half of the fused GEMM + reduce-scatter: rank-order sum of the partial tiles every rank's GEMM
        epilogue pushed here, all-gather of the bf16 result into ``out[:n_rows]`` on every rank."""
        assert out.is_contiguous() and out.dtype == torch.bfloat16
        rc = self.L.vg_comm_gemm_rs_finish(ctypes.byref(self.ctx), ptr(out), c_int(n_rows), c_int(out.shape[1]),
                                           c_int(rs_rows), stream())
        _lib.check(rc, "vg_comm_gemm_rs_finish")

    def ag_gemm(self, q, x_shard: torch.Tensor, row0: int, n_total: int, out: torch.Tensor) -> torch.Tensor:
        """Fused all-gather + GEMM: ``x_shard`` (f16 ``[rows, K]``, this rank's token rows starting at the
        128-aligned ``row0``) is pushed into every rank's landing zone; the GEMM over all ``n_total`` rows reads the
        zone tile by tile as the tiles arrive. Needs ``ag_bytes`` >= 2 * n_total * K * 2 at construction."""
        from ..ops import gemm as G
        K_ = x_shard.shape[1]
        assert x_shard.dtype == torch.float16 and x_shard.is_contiguous() and self.agbuf_bytes > 0
        rc = self.L.vg_comm_ag_push(ctypes.byref(self.ctx), ptr(x_shard), c_int(row0), c_int(x_shard.shape[0]), c_int(K_),
                                    stream())
        _lib.check(rc, "vg_comm_ag_push")
        cap_rows = (self.agbuf_bytes // 2 // (K_ * 2)) // 128 * 128
        zone = self._view(self.agbuf_off, 2 * cap_rows * K_, torch.float16).view(2 * cap_rows, K_)
        return G.linear(q, zone, n_total, out=out, comm=self, ag=True)

    def all_gather_small(self, t: torch.Tensor) -> torch.Tensor:
        """[world, ...] stack of a small contiguous tensor from every rank."""
        out = torch.empty((self.world,) + tuple(t.shape), dtype=t.dtype, device=t.device)
        if self.use_nccl:
            dist.all_gather_into_tensor(out, t.contiguous(), group=self.group)
            return out
        rc = self.L.vg_comm_allgather_small(ctypes.byref(self.ctx), ptr(t), ptr(out), c_int(t.numel() * t.element_size()),
                                            stream())
        _lib.check(rc, "vg_comm_allgather_small")
        return out

    def argmax_merge(self, val: torch.Tensor, idx: torch.Tensor, n: int, out: torch.Tensor):
        """Global arg-max from per-rank (value, global index) pairs; enqueue-only (graph capturable)."""
        assert 1 <= n <= ARGMAX_MAX_COLS, f"arg-max merge handles at most {ARGMAX_MAX_COLS} columns, got {n}"
        rc = self.L.vg_comm_argmax_merge(ctypes.byref(self.ctx), ptr(val), ptr(idx), c_int(n), ptr(self._pairs),
                                         ptr(self._gathered), ptr(out), stream())
        _lib.check(rc, "vg_comm_argmax_merge")

    def argmax_vocab_parallel(self, logits: torch.Tensor) -> List[int]:
        """Greedy token per row from vocabulary-sharded fp32 logits ``[n, V_local]``."""
        from ..ops import kernels as K
        n, vl = logits.shape
        assert 1 <= n <= ARGMAX_MAX_COLS, f"arg-max merge handles at most {ARGMAX_MAX_COLS} columns, got {n}"
        lg = logits if logits.dtype == torch.float32 else logits.float()
        K.argmax(lg, n, self._idx, self._val, idx_offset=self.rank * vl)
        if self.use_nccl:
            pairs = torch.stack([self._val[:n], self._idx[:n].float()], -1)
            allp = self.all_gather_small(pairs)
            best = allp[..., 0].argmax(0)       # first maximum = lowest rank = lowest index
            return [int(allp[int(best[c]), c, 1]) for c in range(n)]
        self.argmax_merge(self._val, self._idx, n, self._out_tok)
        return self._out_tok[:n].tolist()

    def gather_logits(self, logits: torch.Tensor) -> torch.Tensor:
        """Full ``[n, V]`` logits from vocabulary shards (library all-gather; sampling paths only)."""
        n, vl = logits.shape
        out = torch.empty((self.world, n, vl), dtype=logits.dtype, device=logits.device)
        dist.all_gather_into_tensor(out, logits.contiguous(), group=self.group)
        return out.permute(1, 0, 2).reshape(n, self.world * vl)

    # ------------------------------------------------------------ health
    def check(self):
        v = int(self._status_view.item())
        if v != 0:
            self._status_view.zero_()
            raise CommError(f"peer-memory collective reported error {v} (4 = a peer's flag did not arrive in time)")

    def wait_timeout_probe(self, budget_s: float = 0.05):
        """Runs a wait nothing will satisfy; afterwards ``check()`` must raise. Test hook for the bounded-wait path."""
        rc = self.L.vg_comm_wait_timeout_probe(ctypes.byref(self.ctx), ctypes.c_ulonglong(int(budget_s * 1e9)), stream())
        _lib.check(rc, "vg_comm_wait_timeout_probe")

    def barrier(self):
        dist.barrier(group=self.group)

"""GPU model runtime: weights on device, slotted KV / GDN-state store, and the layer loop that drives
the sm_100a kernels for decode, width-N verify and prefill, with CUDA-graph capture of the decode step.

It plays the role of the reference's ``GpuModel`` (reference: src/gpu.rs:3635-3698 layer loop,
:3451-3597 mixers, :3143-3163 FFN, :4132-4259 state, :3987-4081 graphs) with a different shape:
token-major activations, one fused residual+norm kernel between GEMMs, f16 GEMM inputs produced by the
preceding kernel, and a single column-metadata plan (slot / parent / checkpoint arrays) shared by
decode, chain, tree and forest verify and prefill.
"""
from __future__ import annotations

import os
import sys
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..config import ModelConfig
from ..ops import gemm as G
from ..ops import kernels as K
from ..ops import lib as _lib
from .weights import LayerW, ModelWeights, MoeW, QLinear

MTP_GRAPH_MAX_COLS = 8        # draft-head calls of at most this many columns are captured (one graph per width)
MAX_PATH = 16


@dataclass
class Plan:
    """Host-side description of the columns of one forward call."""
    tok: List[int]
    pos: List[int]                      # RoPE position of each column
    kv_slot: List[int]
    kv_row: List[int]                   # cache row the column's K/V are written to
    lens: List[int]                     # number of keys the column attends to
    base: List[int]                     # keys below base[c] are rows 0..base-1; the rest come from path
    path: List[List[int]]               # extra rows per column (tree / forest), at most MAX_PATH
    st_in: List[int]
    parent: List[int]
    st_out: List[int]
    chains: List[Tuple[int, int]]       # (start, length) of sequentially dependent column runs
    direct_attn: bool = False           # prefill: single split, merge fused

    @property
    def n(self) -> int:
        return len(self.tok)

    # ---- constructors
    @staticmethod
    def decode(tokens, pos, slots) -> "Plan":
        n = len(tokens)
        return Plan(list(tokens), list(pos), list(slots), list(pos), [p + 1 for p in pos], [p + 1 for p in pos],
                    [[] for _ in range(n)], list(slots), [-1] * n, list(slots), [(i, 1) for i in range(n)])

    @staticmethod
    def chain(slot, tokens, pos_start, ckpt_base: Optional[int], final_to_slot: bool = False,
              direct_attn: bool = False) -> "Plan":
        n = len(tokens)
        pos = [pos_start + t for t in range(n)]
        st_out = [(-1 if ckpt_base is None else ckpt_base + t) for t in range(n)]
        if final_to_slot:
            st_out[-1] = slot
        return Plan(list(tokens), pos, [slot] * n, pos, [p + 1 for p in pos], [p + 1 for p in pos],
                    [[] for _ in range(n)], [slot] * n, [t - 1 for t in range(n)], st_out, [(0, n)], direct_attn)

    @staticmethod
    def tree(slot, tokens, pos_start, ckpt_base, parent) -> "Plan":
        n = len(tokens)
        depth, paths = [0] * n, []
        for t in range(n):
            p = parent[t]
            paths.append(([] if p < 0 else paths[p]) + [pos_start + t])
            depth[t] = 0 if p < 0 else depth[p] + 1
        return Plan(list(tokens), [pos_start + d for d in depth], [slot] * n, [pos_start + t for t in range(n)],
                    [pos_start + len(paths[t]) for t in range(n)], [pos_start] * n, paths, [slot] * n,
                    list(parent), [ckpt_base + t for t in range(n)], [(0, n)])

    @staticmethod
    def concat(plans: Sequence["Plan"]) -> "Plan":
        """Pack several lanes' plans into one forward (forest verify)."""
        out = Plan([], [], [], [], [], [], [], [], [], [], [])
        for p in plans:
            off = out.n
            out.chains += [(s + off, l) for s, l in p.chains]
            out.parent += [(-1 if q < 0 else q + off) for q in p.parent]
            out.tok += p.tok; out.pos += p.pos; out.kv_slot += p.kv_slot; out.kv_row += p.kv_row
            out.lens += p.lens; out.base += p.base; out.path += p.path
            out.st_in += p.st_in; out.st_out += p.st_out
        return out


class Workspace:
    """Persistent device buffers for up to ``cap`` columns (fixed addresses, so forwards over them can be
    captured in a CUDA graph)."""

    def __init__(self, cfg: ModelConfig, w: ModelWeights, cap: int, device, logits_rows: int):
        c = cfg
        self.cap = cap
        rows = max(cap, 16)
        dev = device
        i32 = lambda *s: torch.zeros(s, dtype=torch.int32, device=dev)
        bf = lambda *s: torch.zeros(s, dtype=torch.bfloat16, device=dev)
        f16 = lambda *s: torch.zeros(s, dtype=torch.float16, device=dev)
        f32 = lambda *s: torch.zeros(s, dtype=torch.float32, device=dev)
        # all per-column int32 metadata lives in one buffer so a step needs a single host->device copy
        self.meta = i32(11, rows)
        self.meta_host = torch.zeros((11, rows), dtype=torch.int32).pin_memory()
        self.meta_host_np = self.meta_host.numpy()        # same pinned memory, written without tensor constructors
        (self.tok, self.pos, self.kv_slot, self.kv_row, self.lens, self.base, self.st_in, self.parent, self.st_out,
         self.chain_start, self.chain_len) = [self.meta[i] for i in range(11)]
        self.path = i32(rows, MAX_PATH)
        h = c.hidden_size
        self.x = bf(rows, h)
        self.xn16 = f16(rows, h)
        self.delta = bf(rows, h)
        widths = [1]
        for L in list(w.layers) + ([w.mtp.layer] if w.mtp else []):
            if L.attn:
                widths.append(L.attn.qkv.m)
            if L.gdn:
                widths.append(L.gdn.in_proj.m)
            if L.mlp:
                widths.append(L.mlp.gate_up.m)
            if L.moe and L.moe.shared:
                widths.append(L.moe.shared.gate_up.m)
        self.wide = bf(rows, (max(widths) + 63) // 64 * 64)                 # qkv / in_proj / gate_up outputs
        self._a16 = {}                                    # contiguous f16 GEMM-input buffers by width
        self._rows, self._dev = rows, dev
        nh_max = max([L.attn.nh for L in list(w.layers) + ([w.mtp.layer] if w.mtp else []) if L.attn] or [1])
        self.q = bf(rows, nh_max * c.head_dim)
        conv_max = max([L.gdn.conv_w.shape[0] for L in w.layers if L.gdn] or [1])
        self.conv_out = f32(rows, conv_max)
        self.logits = f32(max(logits_rows, 1), w.lm_head.m)
        self.out_tok = i32(rows)
        self.out_val = f32(rows)
        self.hidden_keep = bf(rows, h)
        if w.mtp is not None:
            self.cat16 = f16(rows, 2 * h)
            self.mtp_e = bf(rows, h)
        self.n_uploaded = 0
        self.upload_done = None

    def a16(self, width: int) -> torch.Tensor:
        """Contiguous f16 ``[rows, width]`` buffer that receives attention / GDN / SwiGLU outputs."""
        t = self._a16.get(width)
        if t is None:
            t = torch.zeros((self._rows, width), dtype=torch.float16, device=self._dev)
            self._a16[width] = t
        return t


class GpuModel:
    def __init__(self, weights: ModelWeights, device="cuda", max_cols: int = 16, prefill_chunk: int = 4096,
                 comm=None, keep_canonical: bool = False):
        self.w = weights
        self.cfg = weights.cfg
        self.dev = torch.device(device)
        self.comm = comm
        self.max_cols = max_cols
        self.prefill_chunk = prefill_chunk
        self.fuse_allreduce = os.environ.get("VELO_NO_FUSED_ALLREDUCE", "0") != "1"
        # decode / verify widths run NVFP4 linears on the block-scaled FP4 tensor-core kernel
        self.use_fp4 = os.environ.get("VELO_NO_FP4_MMA", "0") != "1"
        # tensor-parallel decode: row-parallel GEMMs push partial rows, the following norm kernel sums them
        self.split_allreduce = os.environ.get("VELO_NO_SPLIT_ALLREDUCE", "0") != "1"
        self._pending_ar = 0                  # 0 none, 1 pair slots, 2 multimem slots hold the pending partial rows
        # --prefill-scalar: exact per-token prefill kernels only (bit-identical to stepping the decode kernels)
        self.prefill_exact = os.environ.get("VELO_PREFILL_SCALAR", "0") == "1"
        self.tc_prefill_attn = os.environ.get("VELO_NO_TC_PREFILL_ATTN", "0") != "1" and not self.prefill_exact
        # decode / verify attention on the tensor cores (head_dim 256, bf16 cache, no tree paths); the CUDA-core
        # split kernel serves every other case
        self.mtp_graphs = os.environ.get("VELO_NO_DECODE_GRAPHS", "0") != "1"    # draft-head steps as graph replays
        self.debug_hash = os.environ.get("VELO_DEBUG_HASH", "0") == "1"
        self.cap_debug = os.environ.get("VELO_CAP_DEBUG", "0") == "1"
        self.tc_decode_attn_default = os.environ.get("VELO_TC_DECODE_ATTN", "1") == "1"
        self.tc_decode_attn = self.tc_decode_attn_default
        self._prefill_ctx = None              # (slot, first position) while a prefill chunk is running
        self.kv_q4 = os.environ.get("VELO_KV_QUANT", "bf16").lower() == "q4"
        self._kv_scales = None                # (k scales, v scales) of the layer being run, 4-bit cache only
        self._gdn_o = None                    # fp32 raw outputs of the column-split / chunked GDN prefill kernels
        self._gdn_work = None                 # operand images handed between the two chunked GDN prefill kernels
        self.gdn_chunk_min = int(os.environ.get("VELO_GDN_CHUNK_MIN", "128"))   # shorter prefill chunks run the exact kernel
        self._k_rows = None                   # bf16 staging of a lane's keys for tensor-core prefill over a 4-bit cache
        # MoE decode: second stream for the shared expert (see moe_runtime.moe_forward)
        self.moe_side_stream = None
        if os.environ.get("VELO_NO_MOE_FORK", "0") != "1" and any(L.moe is not None for L in weights.layers):
            with torch.cuda.device(self.dev):
                self.moe_side_stream = torch.cuda.Stream()
                self.moe_fork_event = torch.cuda.Event()
                self.moe_join_event = torch.cuda.Event()
        self._vt = None
        _lib.lib()
        # FR-Spec: the draft head scores a subset of the vocabulary (rows of the real head: exact)
        self.draft_head = None
        self.draft_ids = None
        dv = int(os.environ.get("VELO_DRAFT_VOCAB", "65536"))
        head = weights.lm_head
        if dv > 0 and weights.mtp is not None and (comm is None or comm.world == 1) and head.m > 2 * dv \
                and (head.packed is not None or head.codes is not None or head.w is not None):
            from .weights import draft_vocab_rows, fuse_rows
            top, tail_start = draft_vocab_rows(dv, head.m)
            if top + (head.m - tail_start) < head.m:
                self.draft_head = fuse_rows([head.rows(0, top), head.rows(tail_start, head.m)])
                self.draft_ids = torch.cat([torch.arange(0, top), torch.arange(tail_start, head.m)]).to(self.dev)
        with torch.cuda.device(self.dev):
            if self.draft_head is not None:
                if self.use_fp4 and self.draft_head.fmt == "nvfp4":
                    G.prepare_fp4(self.draft_head)
                G.prepare(self.draft_head, keep_canonical=False)
            for name, q in weights.linears():
                if q.packed is None and q.codes is None and q.w is None:
                    continue
                small = q.m < 128 or name.endswith(("router", "shared_gate"))
                if name == "embed":
                    if weights.lm_head is weights.embed:
                        if self.use_fp4 and q.fmt == "nvfp4" and q.packed is not None:
                            G.prepare_fp4(q)
                        G.prepare(q, keep_canonical=True)
                    continue
                if small and q.experts <= 1 and q.w is not None and name.endswith(("router", "shared_gate")):
                    G.prepare(q, keep_canonical=True)        # f16 tiles for prefill widths; decode keeps the GEMV
                    continue
                if small or q.experts > 1:
                    continue
                if self.use_fp4 and q.fmt == "nvfp4" and q.packed is not None:
                    G.prepare_fp4(q)
                G.prepare(q, keep_canonical=keep_canonical)
        self.ws = Workspace(self.cfg, weights, max_cols, self.dev, max_cols)
        # token selection on the device (penalties, top-k, nucleus, draw, speculative accept), vocabulary-shard aware
        from ..engine.device_sampler import DeviceSampler
        self.sampler = DeviceSampler(self.dev, weights.lm_head.m, cap=max(16, max_cols), comm=comm)
        # False: forwards return this rank's vocabulary shard of the logits (the device sampler merges shards itself)
        self.gather_logits = True
        self.col_ctr = torch.zeros(48, dtype=torch.int32, device=self.dev)     # per column: two counters, running maximum
        self.ws_prefill: Optional[Workspace] = None
        self.state_ready = False
        self.graphs: Dict[Tuple[str, int], torch.cuda.CUDAGraph] = {}
        self.ns_grid = 32

    # ---------------------------------------------------------------- state
    def alloc_state(self, n_slots: int, n_state_slots: int, max_seq: int):
        c = self.cfg
        dev = self.dev
        if getattr(self, "state_ready", False) and (self.n_slots, self.n_state_slots, self.max_seq) == (n_slots, n_state_slots, max_seq) \
                and self._state_kv_q4 == self.kv_q4:
            # the same shape again (a new scheduler over this runner): clear the state in place and keep the buffers, so
            # the captured graphs, which hold their addresses, stay valid
            for t in [self.S, self.conv, getattr(self, "mtp_kc", None), getattr(self, "mtp_vc", None), self.mtp_ks,
                      self.mtp_vs] + self._kv_tensors():
                if t is not None:
                    t.zero_()
            return
        self._state_kv_q4 = self.kv_q4
        self.n_slots, self.n_state_slots, self.max_seq = n_slots, n_state_slots, max_seq
        attn_layers = [i for i, L in enumerate(self.w.layers) if L.attn]
        gdn_layers = [i for i, L in enumerate(self.w.layers) if L.gdn]
        self.attn_index = {li: j for j, li in enumerate(attn_layers)}
        self.gdn_index = {li: j for j, li in enumerate(gdn_layers)}
        nkv = self.w.layers[attn_layers[0]].attn.nkv if attn_layers else 1
        hd = c.head_dim
        self.ks = self.vs = self.mtp_ks = self.mtp_vs = None
        if self.kv_q4:
            # 4-bit cache: code bytes (two per byte) + one f16 scale per 16 values, 5 bits per value
            assert hd % 32 == 0
            self.kc = torch.zeros((len(attn_layers), n_slots, nkv, max_seq, hd // 2), dtype=torch.uint8, device=dev)
            self.ks = torch.zeros((len(attn_layers), n_slots, nkv, max_seq, hd // 16), dtype=torch.float16, device=dev)
            self.vc, self.vs = torch.zeros_like(self.kc), torch.zeros_like(self.ks)
        else:
            self.kc = torch.zeros((len(attn_layers), n_slots, nkv, max_seq, hd), dtype=torch.bfloat16, device=dev)
            self.vc = torch.zeros_like(self.kc)
        if gdn_layers:
            g0 = self.w.layers[gdn_layers[0]].gdn
            self.S = torch.zeros((len(gdn_layers), n_state_slots, g0.nv, c.lin_k_dim, c.lin_v_dim),
                                 dtype=torch.float32, device=dev)
            self.conv = torch.zeros((len(gdn_layers), n_state_slots, g0.conv_w.shape[0], c.conv_kernel),
                                    dtype=torch.float32, device=dev)
        else:
            self.S = self.conv = None
        if self.w.mtp is not None:
            mn = self.w.mtp.layer.attn.nkv
            if self.kv_q4:
                self.mtp_kc = torch.zeros((n_slots, mn, max_seq, hd // 2), dtype=torch.uint8, device=dev)
                self.mtp_ks = torch.zeros((n_slots, mn, max_seq, hd // 16), dtype=torch.float16, device=dev)
                self.mtp_vc, self.mtp_vs = torch.zeros_like(self.mtp_kc), torch.zeros_like(self.mtp_ks)
            else:
                self.mtp_kc = torch.zeros((n_slots, mn, max_seq, hd), dtype=torch.bfloat16, device=dev)
                self.mtp_vc = torch.zeros_like(self.mtp_kc)
        nh = max([L.attn.nh for L in self.w.layers if L.attn] + ([self.w.mtp.layer.attn.nh] if self.w.mtp else []) or [1])
        self.attn_part = torch.zeros(K.attn_scratch_floats(max(self.max_cols, 16), nh, c.head_dim, self.ns_grid),
                                     dtype=torch.float32, device=dev)
        self.state_ready = True
        self.graphs.clear()

    def copy_state(self, src: int, dst: int):
        if self.S is not None:
            self.S[:, dst].copy_(self.S[:, src])
            self.conv[:, dst].copy_(self.conv[:, src])

    def zero_slot(self, slot: int, zero_kv: bool = False):
        if self.S is not None:
            self.S[:, slot].zero_()
            self.conv[:, slot].zero_()
        if zero_kv:
            for t in self._kv_tensors():
                t[:, slot].zero_()

    def compact_kv(self, slot: int, pos_start: int, cols: Sequence[int]):
        """Move KV rows of accepted tree columns to contiguous positions (reference: src/gpu.rs:5325-5414)."""
        src = torch.tensor([pos_start + c_ for c_ in cols], device=self.dev)
        dst = torch.arange(pos_start, pos_start + len(cols), device=self.dev)
        for cache in self._kv_tensors():
            rows = cache[:, slot].index_select(2, src)
            cache[:, slot].index_copy_(2, dst, rows)

    def _kv_tensors(self):
        """Main-model cache tensors, all shaped [attention layer, slot, kv head, position, ...]."""
        return [t for t in (self.kc, self.vc, self.ks, self.vs) if t is not None]

    # ---------------------------------------------------------------- health
    def health_check(self):
        """Per-step failure probe without a synchronisation of its own: the kernels' bounded-wait status word and
        the communicator's status word are copied to pinned host memory asynchronously; each call first reads the
        copy the previous call enqueued (complete by now: the step's token read synchronised the stream in
        between) and raises ``KernelError`` / ``CommError`` when either word is non-zero. Plays the role of the
        reference's transport watchdog + abort word (reference: native/net_shim.c:471-507, src/main.rs:2825-2858)."""
        if getattr(self, "_health_host", None) is None:
            self._health_host = torch.zeros(2, dtype=torch.int32).pin_memory()
            self._health_dev = torch.zeros(2, dtype=torch.int32, device=self.dev)
            self._health_evt = None
        if self._health_evt is not None and self._health_evt.query():
            kerr, cerr = int(self._health_host[0]), int(self._health_host[1])
            if kerr or cerr:
                self._health_host.zero_()
                _lib.err_word(self.dev).zero_()
                if self.comm is not None and self.comm.world > 1:
                    self.comm._status_view.zero_()
                if cerr:
                    from ..parallel.comm import CommError
                    raise CommError(f"peer-memory collective reported error {cerr} (4 = a peer's flag did not arrive in time)")
                raise _lib.KernelError(f"a kernel reported bounded-wait failure code {kerr}")
        self._health_dev[0:1].copy_(_lib.err_word(self.dev))
        if self.comm is not None and self.comm.world > 1:
            self._health_dev[1:2].copy_(self.comm._status_view)
        self._health_host.copy_(self._health_dev, non_blocking=True)
        if self._health_evt is None:
            self._health_evt = torch.cuda.Event()
        self._health_evt.record()

    # ---------------------------------------------------------------- plan upload
    def _upload(self, ws: Workspace, p: Plan):
        n = p.n
        assert n <= ws.cap, (n, ws.cap)
        cs = [s for s, _ in p.chains] + [0] * (n - len(p.chains))
        cl = [l for _, l in p.chains] + [0] * (n - len(p.chains))
        # one numpy conversion for the eleven per-column rows (a tensor constructor per row costs tens of microseconds
        # of host time on every step)
        rows = np.asarray((p.tok, p.pos, p.kv_slot, p.kv_row, p.lens, p.base, p.st_in, p.parent, p.st_out, cs, cl), dtype=np.int32)
        # a plan that names a cache row, lane or state slot outside the allocated state would write through it
        if rows[3].max() >= self.max_seq or rows[4].max() > self.max_seq or rows[2].max() >= self.n_slots \
                or max(rows[6].max(), rows[8].max()) >= self.n_state_slots or rows[3].min() < 0 or rows[2].min() < 0:
            raise ValueError(f"plan outside the allocated state: rows <= {rows[3].max()} of {self.max_seq}, lanes <= "
                             f"{rows[2].max()} of {self.n_slots}, state slots <= {max(rows[6].max(), rows[8].max())} of "
                             f"{self.n_state_slots}")
        if ws.upload_done is not None:
            ws.upload_done.synchronize()        # the previous copy must have left the pinned buffer
        ws.meta_host_np[:, :n] = rows
        mh = ws.meta_host
        if mh.shape[1] <= 64:
            ws.meta.copy_(mh, non_blocking=True)
        else:
            ws.meta[:, :n].copy_(mh[:, :n], non_blocking=True)
        if any(p.path):
            path = [row + [0] * (MAX_PATH - len(row)) for row in p.path]
            ws.path[:n].copy_(torch.tensor(path, dtype=torch.int32), non_blocking=True)
        if ws.upload_done is None:
            ws.upload_done = torch.cuda.Event()
        ws.upload_done.record()
        ws.n_uploaded = n

    # ---------------------------------------------------------------- layers
    def _reduce(self, t: torch.Tensor, n: int):
        if self.comm is not None and self.comm.world > 1:
            self.comm.all_reduce_rows(t, n)

    def _fp4_ok(self, q: QLinear, n: int) -> bool:
        return self.use_fp4 and n <= 16 and getattr(q, "kernel4", None) is not None

    def _norm(self, ws: Workspace, delta, w: torch.Tensor, n: int):
        """Residual add + RMSNorm into ``ws.xn16``; at decode widths the same kernel also emits the FP4
        activation series, returned for the linears that read this input. When the preceding row-parallel
        linear only pushed its partial rows (``self._pending_ar``), the kernel also performs the
        tensor-parallel sum."""
        if self._pending_ar:
            mode, self._pending_ar = self._pending_ar, 0
            return G.add_rmsnorm_fp4_ar(ws.x, w, self.cfg.rms_eps, n, self.comm, out16=ws.xn16, mode=mode)
        if self.use_fp4 and n <= 16 and ws.x.shape[1] % 16 == 0:
            return G.add_rmsnorm_fp4(ws.x, delta, w, self.cfg.rms_eps, n, out16=ws.xn16)
        K.add_rmsnorm(ws.x, delta, w, self.cfg.rms_eps, n, out16=ws.xn16)
        return None

    def _linear(self, q: QLinear, x16: torch.Tensor, n: int, out: torch.Tensor, act=None, out_f32: bool = False,
                comm=None):
        if self._fp4_ok(q, n):
            G.linear_fp4(q, x16, n, out=out, out_f32=out_f32, comm=comm, act=act)
        else:
            G.linear(q, x16, n, out=out, out_f32=out_f32, comm=comm)

    def _row_parallel(self, q: QLinear, x16: torch.Tensor, n: int, out: torch.Tensor, reduce: bool = True, act=None):
        """Row-parallel linear + tensor-parallel sum. For decode / verify widths the reduction is fused into
        the GEMM epilogue (peer-memory pushes + flags inside the same kernel); longer inputs run the GEMM and
        then the two-shot peer-memory all-reduce."""
        tp = reduce and self.comm is not None and self.comm.world > 1
        if tp and n <= 16 and not self.comm.use_nccl and self.fuse_allreduce and (q.m + 127) // 128 <= 64:
            # (a reduced row-parallel output is always the delta the next residual-add / RMSNorm consumes)
            if self.split_allreduce and self._fp4_ok(q, n) and q.m == self.cfg.hidden_size and q.m % 16 == 0:
                # push the partial rows; the next residual-add / RMSNorm kernel sums them
                G.linear_fp4(q, x16, n, out=out, comm=self.comm, act=act, push_only=True)
                self._pending_ar = 2 if self.comm.use_mm else 1       # which form the consumer must read
                return
            self._linear(q, x16, n, out, act=act, comm=self.comm)
            return
        if tp and n > 64 and not self.comm.use_nccl and out.dtype == torch.bfloat16 and self.comm.multicast_address(out):
            # prefill widths with a multicast-bound output buffer: plain GEMM, then the in-switch all-reduce in place
            # (measured faster than pushing fp32 partial tiles from the GEMM epilogue: the switch adds the ranks'
            # copies while each element crosses a GPU's links once)
            self._linear(q, x16, n, out, act=act)
            self.comm.all_reduce_rows(out, n)
            return
        if tp and n > 64 and not self.comm.use_nccl and self.fuse_allreduce and out.dtype == torch.bfloat16 \
                and out.is_contiguous() and out.shape[1] == q.m:
            # prefill widths: GEMM fused with the reduce-scatter (each partial tile goes to the rank owning its token
            # rows as soon as it is computed), then the rank-order sum + all-gather
            rs_rows = self.comm.rs_rows_for(n, q.m)
            if rs_rows:
                G.linear(q, x16, n, out=out, comm=self.comm, rs_rows=rs_rows)
                self.comm.gemm_rs_finish(out, n, rs_rows)
                return
        self._linear(q, x16, n, out, act=act)
        if tp:
            self._reduce(out, n)

    def _vt_scratch(self, nkv: int, max_seq: int) -> torch.Tensor:
        """Transposed-value scratch ``[nkv, head_dim, keys]`` of the lane being prefilled (shared by all layers)."""
        cap = (max_seq + 127) // 128 * 128
        if self._vt is None or self._vt.shape[0] < nkv or self._vt.shape[2] != cap:
            self._vt = torch.zeros((nkv, self.cfg.head_dim, cap), dtype=torch.bfloat16, device=self.dev)
        return self._vt[:nkv]

    def _attn(self, ws: Workspace, L: LayerW, n: int, kc, vc, plan_direct: bool, use_path: bool, act=None):
        c, A = self.cfg, L.attn
        qkv = ws.wide[:, :A.qkv.m]
        self._linear(A.qkv, ws.xn16, n, qkv, act=act)
        ksc, vsc = self._kv_scales if self._kv_scales is not None else (None, None)
        K.attn_prep(qkv, A.q_norm, A.k_norm, ws.pos, ws.kv_slot, ws.kv_row, ws.q, kc, vc, n, A.nh, A.nkv,
                    c.head_dim, c.rotary_dim, c.rms_eps, c.rope_theta, c.attn_out_gate, k_scale=ksc, v_scale=vsc)
        a16 = ws.a16(A.o.k)
        pf = self._prefill_ctx
        if plan_direct and pf is not None and n >= 64 and c.head_dim == 256 and self.tc_prefill_attn \
                and qkv.stride(0) % 8 == 0:
            # prefill chunk of one lane: tensor-core flash attention over the lane's cache rows
            slot, pos0 = pf
            k_rows = None
            if ksc is not None:
                if self._k_rows is None or self._k_rows.shape[1] < A.nkv or self._k_rows.shape[2] != kc.shape[2]:
                    self._k_rows = torch.zeros((1, A.nkv, kc.shape[2], c.head_dim), dtype=torch.bfloat16, device=self.dev)
                k_rows = self._k_rows
            K.attn_prefill_tc(ws.q, kc, vc, self._vt_scratch(A.nkv, kc.shape[2]), slot, pos0, n, A.nh, A.nkv, c.head_dim,
                              a16, gate=qkv if c.attn_out_gate else None, k_scale=ksc, v_scale=vsc, k_rows=k_rows)
        elif (self.tc_decode_attn and not plan_direct and not use_path and ksc is None and c.head_dim == 256
              and A.nh // A.nkv <= 16 and n <= 16):
            K.attn_decode_tc(ws.q, kc, vc, ws.lens, ws.kv_slot, self.attn_part, a16, n, A.nh, A.nkv, c.head_dim,
                             gate=qkv if c.attn_out_gate else None, ns_grid=self.ns_grid)
        else:
            K.attn_decode(ws.q, kc, vc, ws.lens, ws.kv_slot, self.attn_part, a16, n, A.nh, A.nkv, c.head_dim,
                          gate=qkv if c.attn_out_gate else None, base=ws.base if use_path else None,
                          path=ws.path if use_path else None, ns_grid=self.ns_grid, direct=plan_direct,
                          k_scale=ksc, v_scale=vsc)
        self._row_parallel(A.o, a16, n, ws.delta)

    def _gdn(self, ws: Workspace, L: LayerW, li: int, n: int, n_chains: int, seq_mode: bool, act=None):
        c, Gd = self.cfg, L.gdn
        linear_chain = seq_mode and n_chains == 1 and ws is self.ws_prefill      # prefill plans are one linear chain
        gi = self.gdn_index[li]
        proj = ws.wide[:, :Gd.in_proj.m]
        conv_dim = Gd.conv_w.shape[0]
        value_dim = Gd.nv * c.lin_v_dim
        if self._fp4_ok(Gd.in_proj, n) and c.conv_kernel <= 8:
            # the conv runs in the GEMM epilogue: each output row is one conv channel
            cv = G.ConvEpi.make(self.conv[gi], Gd.conv_w, ws.st_in, ws.parent, ws.st_out, ws.conv_out, conv_dim,
                                c.conv_kernel)
            G.linear_fp4(Gd.in_proj, ws.xn16, n, out=proj, act=act, conv=cv)
        elif seq_mode:
            self._linear(Gd.in_proj, ws.xn16, n, proj, act=act)
            if not (linear_chain and K.gdn_conv_chain(proj, self.conv[gi], Gd.conv_w, ws.st_in, ws.parent, ws.st_out,
                                                      ws.conv_out, n, conv_dim, c.conv_kernel)):
                K.gdn_conv(proj, self.conv[gi], Gd.conv_w, ws.st_in, ws.parent, ws.st_out, ws.conv_out, n, conv_dim,
                           c.conv_kernel, phase=1)
                K.gdn_conv(proj, self.conv[gi], Gd.conv_w, ws.st_in, ws.parent, ws.st_out, ws.conv_out, n, conv_dim,
                           c.conv_kernel, phase=2)
        else:
            self._linear(Gd.in_proj, ws.xn16, n, proj, act=act)
            K.gdn_conv(proj, self.conv[gi], Gd.conv_w, ws.st_in, ws.parent, ws.st_out, ws.conv_out, n, conv_dim,
                       c.conv_kernel, phase=3)
        g16 = ws.a16(Gd.out.k)
        act_o = None
        if self._fp4_ok(Gd.out, n) and value_dim % 16 == 0:
            # the recurrence kernel quantises its own output rows for the output projection
            act_o = G.fp4_buffers(self.dev, Gd.out.kernel4.kp)
        if linear_chain and n >= self.gdn_chunk_min and c.lin_k_dim == 128 and c.lin_v_dim == 128 and conv_dim % 4 == 0 \
                and not self.prefill_exact:
            # long prefill chunk: the chunked (WY) form of the recurrence on the tensor cores; agrees with the exact
            # kernels to tf32 rounding (decode and verify always run the exact step kernel)
            need = ws.cap * value_dim
            if self._gdn_o is None or self._gdn_o.numel() < need:
                self._gdn_o = torch.zeros(need, dtype=torch.float32, device=self.dev)
            wb = K.gdn_chunk_work_bytes(ws.cap, Gd.nv)
            if self._gdn_work is None or self._gdn_work.numel() < wb + 1024:
                self._gdn_work = torch.zeros(wb + 1024, dtype=torch.uint8, device=self.dev)
            off = (-self._gdn_work.data_ptr()) % 1024
            K.gdn_chunk_prefill(ws.conv_out, proj, conv_dim,
                                conv_dim + value_dim, conv_dim + value_dim + Gd.nv, self.S[gi], Gd.A_log, Gd.dt_bias, Gd.norm,
                                0, n, ws.st_in, ws.st_out, g16, Gd.nk, Gd.nv, c.lin_k_dim, c.lin_v_dim, c.rms_eps,
                                self._gdn_work[off:], self._gdn_o)
        elif linear_chain and n > 16 and c.lin_k_dim == 128 and c.lin_v_dim == 128 and proj.stride(0) % 8 == 0 \
                and conv_dim % 8 == 0:
            # prefill chunk: one chain through all n columns
            need = ws.cap * value_dim
            if self._gdn_o is None or self._gdn_o.numel() < need:
                self._gdn_o = torch.zeros(need, dtype=torch.float32, device=self.dev)
            K.gdn_prefill(ws.conv_out, proj, conv_dim, conv_dim + value_dim, conv_dim + value_dim + Gd.nv, self.S[gi],
                          Gd.A_log, Gd.dt_bias, Gd.norm, 0, n, ws.st_in, ws.st_out, g16, Gd.nk, Gd.nv, c.lin_k_dim,
                          c.lin_v_dim, c.rms_eps, o_scratch=self._gdn_o,
                          split=int(os.environ.get("VELO_GDN_PREFILL_SPLIT", "0")))
        else:
            K.gdn_step(ws.conv_out, proj, conv_dim, conv_dim + value_dim, conv_dim + value_dim + Gd.nv, self.S[gi],
                       Gd.A_log, Gd.dt_bias, Gd.norm, ws.chain_start, ws.chain_len, n_chains, ws.st_in, ws.parent,
                       ws.st_out, g16, Gd.nk, Gd.nv, c.lin_k_dim, c.lin_v_dim, c.rms_eps,
                       quant=act_o + (self.col_ctr,) if act_o is not None else None)
        self._row_parallel(Gd.out, g16, n, ws.delta, act=act_o)

    def _mlp(self, ws: Workspace, M, n: int, out: torch.Tensor, reduce: bool = True, act=None, buf_tag: str = ""):
        """SwiGLU MLP. ``buf_tag`` selects a private set of FP4 activation buffers (an MLP that runs on a second
        stream must not share them with the main stream's producers)."""
        gu = ws.wide[:, :M.gate_up.m]
        self._linear(M.gate_up, ws.xn16, n, gu, act=act)
        a16 = ws.a16(M.down.k)
        if self._fp4_ok(M.down, n) and M.inter % 8 == 0:
            bufs = G.fp4_buffers(self.dev, ((M.inter + 255) // 256) * 256, tag=buf_tag) if buf_tag else None
            act_d = G.swiglu_fp4(gu, n, M.inter, bufs=bufs)
            self._row_parallel(M.down, a16, n, out, reduce, act=act_d)
            return
        K.swiglu(gu, a16, n, M.inter)
        self._row_parallel(M.down, a16, n, out, reduce)

    def _moe(self, ws: Workspace, M: MoeW, n: int, act=None):
        from . import moe_runtime
        moe_runtime.moe_forward(self, ws, M, n, act=act)

    def _layer(self, ws, L: LayerW, li, n, n_chains, seq_mode, direct, use_path, kc, vc, first_delta):
        c = self.cfg
        act = self._norm(ws, first_delta, L.input_norm, n)
        if self.cap_debug:
            self._cap_debug(f"layer {li} normed", ws.xn16, n)
        if L.attn is not None:
            self._attn(ws, L, n, kc, vc, direct, use_path, act=act)
        else:
            self._gdn(ws, L, li, n, n_chains, seq_mode, act=act)
        if self.cap_debug and not self._pending_ar:
            self._cap_debug(f"layer {li} mixer out", ws.delta, n)
        act = self._norm(ws, ws.delta, L.post_norm, n)
        if L.moe is not None:
            self._moe(ws, L.moe, n, act=act)
        else:
            self._mlp(ws, L.mlp, n, ws.delta, act=act)
        if self.cap_debug and not self._pending_ar:
            self._cap_debug(f"layer {li} ffn out", ws.delta, n)

    def _backbone(self, ws: Workspace, n: int, n_chains: int, seq_mode: bool, direct: bool, use_path: bool,
                  logits_rows: Optional[Tuple[int, int]] = None):
        """Embedding -> layers -> final norm -> LM head over rows [r0, r1) (default: all n).
        Leaves the pre-final-norm hidden in ws.x and fp32 logits in ws.logits[: r1 - r0]."""
        c = self.cfg
        K.embed_gather(self.w.embed, ws.tok, ws.x, n)
        delta = None
        for li, L in enumerate(self.w.layers):
            kc = vc = None
            if L.attn is not None:
                ai = self.attn_index[li]
                kc, vc = self.kc[ai], self.vc[ai]
                self._kv_scales = (self.ks[ai], self.vs[ai]) if self.kv_q4 else None
            self._layer(ws, L, li, n, n_chains, seq_mode, direct, use_path, kc, vc, delta)
            delta = ws.delta
        act = self._norm(ws, delta, self.w.final_norm, n)
        r0, r1 = (0, n) if logits_rows is None else logits_rows
        if r1 > r0:
            if r0 != 0:
                # the LM head always reads from the start of the buffer (one cached tensor map)
                assert r0 >= r1 - r0
                ws.xn16[:r1 - r0].copy_(ws.xn16[r0:r1])
                act = None
            self._linear(self.w.lm_head, ws.xn16, r1 - r0, ws.logits, act=act, out_f32=True)

    # ---------------------------------------------------------------- public forwards
    def forward(self, plan: Plan, want_logits: bool = True) -> Tuple[Optional[torch.Tensor], torch.Tensor]:
        """Generic forward over the small workspace. Returns (logits [n, V_local] fp32 view, hidden [n, h] bf16 view)."""
        ws = self.ws
        self._upload(ws, plan)
        n = plan.n
        seq_mode = any(l > 1 for _, l in plan.chains)
        self._backbone(ws, n, len(plan.chains), seq_mode, plan.direct_attn, any(plan.path),
                       None if want_logits else (0, 0))
        return (self._full_logits(ws.logits[:n]) if want_logits else None), ws.x[:n]

    def decode(self, tokens, pos, slots):
        return self.forward(Plan.decode(tokens, pos, slots))

    def verify(self, slot, tokens, pos_start, ckpt_base=None, parent=None):
        if parent is None:
            return self.forward(Plan.chain(slot, tokens, pos_start, ckpt_base))
        return self.forward(Plan.tree(slot, tokens, pos_start, ckpt_base, parent))

    def verify_forest(self, lanes):
        """Several lanes' chain verifies packed into one forward of at most ``max_cols`` columns:
        list of (slot, tokens, pos_start, ckpt_base) -> list of (logits, hidden) clones per lane."""
        plans = [Plan.chain(slot, toks, pos, ck) for slot, toks, pos, ck in lanes]
        widths = {pl.n for pl in plans}
        if self.mtp_graphs and len(widths) == 1 and len(plans) * plans[0].n <= self.ws.cap \
                and all(ck is not None for _, _, _, ck in lanes):
            # equal chain widths (what the scheduler packs): one graph per (lanes, width)
            logits, hidden = self._replay_forest(plans, min(ck for _, _, _, ck in lanes))
        else:
            logits, hidden = self.forward(Plan.concat(plans))
        outs, o = [], 0
        for pl in plans:
            outs.append((logits[o:o + pl.n].clone(), hidden[o:o + pl.n].clone()))
            o += pl.n
        return outs

    def prefill(self, slot: int, tokens: Sequence[int], pos_start: int = 0, want_hidden: bool = True):
        """Chunked prefill of one lane; state carried in the lane's slot. Returns (logits of the last
        token [V_local] fp32, hidden [N, h] bf16 or None)."""
        N = len(tokens)
        chunk = min(self.prefill_chunk, max(N, 16))
        if self.ws_prefill is None or self.ws_prefill.cap < chunk:
            self.ws_prefill = Workspace(self.cfg, self.w, chunk, self.dev, 1)
            if self.comm is not None and self.comm.world > 1 and self.comm.mc and not self.comm.use_nccl \
                    and os.environ.get("VELO_NO_MULTIMEM_PREFILL", "0") != "1":
                # the row-parallel outputs of a prefill chunk land in multicast-bound symmetric memory, where the
                # tensor-parallel sum runs in place inside the NVLink switch (collective allocation: every rank
                # creates its prefill workspace at the same point)
                wsp = self.ws_prefill
                buf = self.comm.symmetric_buffer(wsp.delta.numel() * 2)
                if buf is not None:
                    wsp.delta = buf.view(torch.bfloat16).view(wsp.delta.shape)
            need = K.attn_scratch_floats(16, 1, self.cfg.head_dim, 1)
            assert self.attn_part.numel() >= need
        ws = self.ws_prefill
        hs = []
        logits = None
        for o in range(0, N, chunk):
            toks = tokens[o:o + chunk]
            n = len(toks)
            last = o + n >= N
            plan = Plan.chain(slot, toks, pos_start + o, None, final_to_slot=True, direct_attn=True)
            self._upload(ws, plan)
            self._prefill_ctx = (slot, pos_start + o)
            try:
                self._backbone(ws, n, 1, True, True, False, (n - 1, n) if last else (0, 0))
            finally:
                self._prefill_ctx = None
            if want_hidden:
                hs.append(ws.x[:n].clone())
            if last:
                logits = self._full_logits(ws.logits[:1])[0]
        if self.debug_hash:
            self._dbg_probe_prefill(f"prefill.slot{slot}", slot, pos_start + N, ws.x[n - 1:n])
        return logits, (torch.cat(hs, 0) if want_hidden else None)

    # ---------------------------------------------------------------- debugging probes (host side, env-gated)
    def dbg_hash(self, tag: str, t: torch.Tensor):
        """VELO_DEBUG_HASH=1: FNV-1a over the raw bytes of a tensor plus its first values, on stderr. Two runs (or two
        ranks, or two code paths) that should agree bit for bit are compared by diffing these lines; synchronises, so
        it is for hunting a divergence, not for production (reference: src/gpu.rs:6787-6837)."""
        raw = t.detach().contiguous().view(torch.uint8).cpu().numpy().tobytes()
        h = 0xCBF29CE484222325
        for b in raw:
            h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
        first = [round(float(v), 6) for v in t.detach().reshape(-1)[:4].float().cpu()]
        print(f"  [dbghash] {tag} n={t.numel()} fnv={h:016x} first={first}", file=sys.stderr, flush=True)

    def _dbg_probe_prefill(self, tag: str, slot: int, plen: int, last_hidden: torch.Tensor):
        self.dbg_hash(f"{tag}.hidden_last", last_hidden)
        if self.kc is not None and self.kc.numel() and not self.kv_q4:
            # only the rows the prompt wrote: the rest of a lane's cache holds whatever an earlier request left
            self.dbg_hash(f"{tag}.k.L0[:{plen}]", self.kc[0, slot, :, :plen])
            self.dbg_hash(f"{tag}.v.L0[:{plen}]", self.vc[0, slot, :, :plen])
        if self.S is not None and self.S.numel():
            self.dbg_hash(f"{tag}.gdn_state.L0", self.S[0, slot])

    def _cap_debug(self, tag: str, t: torch.Tensor, n: int):
        """VELO_CAP_DEBUG=1: absolute maximum and rms of an activation, to localise a numeric blow-up layer by layer
        (eager steps only; reference: src/gpu.rs:3496-3502, :5899-5926)."""
        if torch.cuda.is_current_stream_capturing():
            return
        v = t[:n].float()
        print(f"  capdbg {tag}: absmax={float(v.abs().max()):.4f} rms={float(v.pow(2).mean().sqrt()):.6f}",
              file=sys.stderr, flush=True)

    # ---------------------------------------------------------------- MTP head
    def mtp_forward(self, slot: int, tokens: Sequence[int], hidden: torch.Tensor, pos: Sequence[int],
                    tok_dev: Optional[torch.Tensor] = None, draft_only: bool = False):
        """Draft head over N (hidden_t, token_{t+1}) pairs of one lane (replicated on every rank).
        Returns (logits [N, V_local] fp32, head hidden [N, h] bf16). ``tok_dev`` (int32 device tensor, N ids) replaces
        ``tokens`` without a host round trip (a draft chain feeds each draft straight into the next step). With
        ``draft_only`` and a draft-vocabulary head the logits returned are the ``[N, Vd]`` draft-vocabulary scores
        (ids through ``self.draft_ids``) and the scatter into full-vocabulary rows is skipped."""
        m, c, ws = self.w.mtp, self.cfg, self.ws
        n = len(tokens)
        plan = Plan.chain(slot, tokens, 0, None)
        plan.pos = list(pos); plan.kv_row = list(pos)
        plan.lens = [p + 1 for p in pos]; plan.base = list(plan.lens)
        self._upload(ws, plan)
        if tok_dev is not None:
            ws.tok[:n].copy_(tok_dev[:n])
        ws.hidden_keep[:n].copy_(hidden[:n])
        # The device work below reads only workspace buffers (token ids, hidden rows, the uploaded plan) and is
        # idempotent (the head's layer is an attention layer: re-running a column rewrites the same cache row), so
        # small widths, the draft step and the re-prime after a verify, run as graph replays.
        if self.mtp_graphs and n <= MTP_GRAPH_MAX_COLS and not torch.cuda.is_current_stream_capturing():
            key = ("mtp", n, bool(draft_only))
            g = self.graphs.get(key)
            if g is None:
                torch.cuda.synchronize(self.dev)
                side = torch.cuda.Stream(device=self.dev)
                side.wait_stream(torch.cuda.current_stream(self.dev))
                with torch.cuda.stream(side):
                    for _ in range(2):
                        self._mtp_body(ws, n, draft_only)
                torch.cuda.current_stream(self.dev).wait_stream(side)
                torch.cuda.synchronize(self.dev)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self._mtp_body(ws, n, draft_only)
                self.graphs[key] = g
            g.replay()
        else:
            self._mtp_body(ws, n, draft_only)
        if self.draft_head is not None:
            return (self._draft_logits[:n] if draft_only else ws.logits[:n]), ws.x[:n]
        return self._full_logits(ws.logits[:n]), ws.x[:n]

    def _mtp_body(self, ws: Workspace, n: int, draft_only: bool):
        """Device part of the draft head over the ``n`` columns staged in the workspace."""
        m, c = self.w.mtp, self.cfg
        h = c.hidden_size
        K.embed_gather(self.w.embed, ws.tok, ws.mtp_e, n)
        K.add_rmsnorm(ws.mtp_e, None, m.norm_embed, c.rms_eps, n, out_bf=ws.x)
        ws.cat16[:n, :h].copy_(ws.x[:n])
        K.add_rmsnorm(ws.hidden_keep, None, m.norm_hidden, c.rms_eps, n, out_bf=ws.x)
        ws.cat16[:n, h:].copy_(ws.x[:n])
        self._linear(m.fc, ws.cat16, n, ws.x)
        comm, self.comm = self.comm, None          # the draft head is unsharded: no reductions
        try:
            self._kv_scales = (self.mtp_ks, self.mtp_vs) if self.kv_q4 else None
            self._layer(ws, m.layer, -1, n, 1, True, False, False, self.mtp_kc, self.mtp_vc, None)
        finally:
            self.comm = comm
        act = self._norm(ws, ws.delta, m.norm, n)
        if self.draft_head is not None:
            # score the draft vocabulary only; every other token gets -inf so arg-max / sampling stay inside it
            if getattr(self, "_draft_logits", None) is None:
                self._draft_logits = torch.zeros((ws.logits.shape[0], self.draft_head.m), dtype=torch.float32, device=self.dev)
            self._linear(self.draft_head, ws.xn16, n, self._draft_logits, act=act, out_f32=True)
            if not draft_only:
                ws.logits[:n].fill_(float("-inf"))
                ws.logits[:n].index_copy_(1, self.draft_ids, self._draft_logits[:n])
            return
        self._linear(self.w.lm_head, ws.xn16, n, ws.logits, act=act, out_f32=True)

    # ---------------------------------------------------------------- vocabulary-parallel head
    @property
    def tp(self) -> int:
        return self.comm.world if self.comm is not None else 1

    def _full_logits(self, local: torch.Tensor) -> torch.Tensor:
        """Under tensor parallelism the LM head is vocabulary-sharded: gather the shards (sampling paths)."""
        if self.tp == 1 or not self.gather_logits:
            return local
        return self.comm.gather_logits(local)

    def _greedy_tail(self, ws: Workspace, b: int):
        """Arg-max over the (possibly sharded) vocabulary into ws.out_tok; enqueue-only."""
        if self.tp == 1:
            K.argmax(ws.logits, b, ws.out_tok, ws.out_val)
        else:
            vl = ws.logits.shape[1]
            K.argmax(ws.logits, b, self.comm._idx, ws.out_val, idx_offset=self.comm.rank * vl)
            self.comm.argmax_merge(ws.out_val, self.comm._idx, b, ws.out_tok)

    # ---------------------------------------------------------------- CUDA graphs
    def capture_decode(self, b: int):
        """Capture the greedy decode step for batch size ``b``: inputs are read from the workspace's
        device arrays, the arg-max token ids land in ``ws.out_tok``."""
        ws = self.ws
        plan = Plan.decode([0] * b, [0] * b, list(range(b)))
        self._upload(ws, plan)
        # warm-up and capture run real steps on slots 0..b-1 at position 0: save what they touch
        saved = [(t, t[:, :b].clone()) for t in (self.S, self.conv) if t is not None]
        kv = self._kv_tensors()
        saved += [(t, t[:, :b, :, :1].clone()) for t in kv]
        # the attention launch grid covers every possible split, so a graph captured here is valid at any position
        torch.cuda.synchronize(self.dev)
        s = torch.cuda.Stream(device=self.dev)
        s.wait_stream(torch.cuda.current_stream(self.dev))
        with torch.cuda.stream(s):
            for _ in range(2):
                self._backbone(ws, b, b, False, False, False)
                self._greedy_tail(ws, b)
        torch.cuda.current_stream(self.dev).wait_stream(s)
        torch.cuda.synchronize(self.dev)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._backbone(ws, b, b, False, False, False)
            self._greedy_tail(ws, b)
        for t, keep in saved:
            if any(t is x for x in kv):
                t[:, :b, :, :1].copy_(keep)
            else:
                t[:, :b].copy_(keep)
        self.graphs[("decode", b)] = g
        return g

    def capture_verify(self, n: int, ckpt_base: int):
        """Capture a chain verify of ``n`` columns of one lane (reference: the verify-width graphs of
        src/batch.rs:566-633). Lane, positions, tokens and checkpoint slots are read from the workspace's device arrays
        at replay; only the width is fixed. Warm-up and capture run real steps on lane 0 at positions 0..n-1 writing the
        checkpoint slots ``ckpt_base ..``: what they touch is saved and put back."""
        ws = self.ws
        self._upload(ws, Plan.chain(0, [0] * n, 0, ckpt_base))
        touched = [0] + list(range(ckpt_base, ckpt_base + n))
        saved = [(t, t[:, touched].clone()) for t in (self.S, self.conv) if t is not None]
        kv = self._kv_tensors()
        saved_kv = [(t, t[:, :1, :, :n].clone()) for t in kv]
        torch.cuda.synchronize(self.dev)
        s = torch.cuda.Stream(device=self.dev)
        s.wait_stream(torch.cuda.current_stream(self.dev))
        with torch.cuda.stream(s):
            for _ in range(2):
                self._backbone(ws, n, 1, True, False, False)
        torch.cuda.current_stream(self.dev).wait_stream(s)
        torch.cuda.synchronize(self.dev)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._backbone(ws, n, 1, True, False, False)
        for t, keep in saved:
            t[:, touched] = keep
        for t, keep in saved_kv:
            t[:, :1, :, :n].copy_(keep)
        self.graphs[("verify", n)] = g
        return g

    def replay_verify(self, slot: int, tokens: Sequence[int], pos_start: int, ckpt_base: int):
        """``verify`` of a linear chain as a graph replay: same kernels, same bits, one launch."""
        n = len(tokens)
        g = self.graphs.get(("verify", n))
        if g is None:
            g = self.capture_verify(n, ckpt_base)
        self._upload(self.ws, Plan.chain(slot, tokens, pos_start, ckpt_base))
        g.replay()
        return self._full_logits(self.ws.logits[:n]), self.ws.x[:n]

    def _replay_forest(self, plans: Sequence[Plan], ckpt_base: int):
        """Several lanes' equal-width chain verifies packed into one forward, as a graph replay. Capture runs real steps
        on lanes 0..p-1 at positions 0..w-1 with checkpoints from ``ckpt_base``: what they touch is saved and put back."""
        ws = self.ws
        p, w = len(plans), plans[0].n
        n = p * w
        key = ("forest", p, w)
        g = self.graphs.get(key)
        if g is None:
            cap_plan = Plan.concat([Plan.chain(l, [0] * w, 0, ckpt_base + l * w) for l in range(p)])
            self._upload(ws, cap_plan)
            touched = list(range(p)) + list(range(ckpt_base, ckpt_base + n))
            saved = [(t, t[:, touched].clone()) for t in (self.S, self.conv) if t is not None]
            kv = self._kv_tensors()
            saved_kv = [(t, t[:, :p, :, :w].clone()) for t in kv]
            torch.cuda.synchronize(self.dev)
            side = torch.cuda.Stream(device=self.dev)
            side.wait_stream(torch.cuda.current_stream(self.dev))
            with torch.cuda.stream(side):
                for _ in range(2):
                    self._backbone(ws, n, p, True, False, False)
            torch.cuda.current_stream(self.dev).wait_stream(side)
            torch.cuda.synchronize(self.dev)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._backbone(ws, n, p, True, False, False)
            for t, keep in saved:
                t[:, touched] = keep
            for t, keep in saved_kv:
                t[:, :p, :, :w].copy_(keep)
            self.graphs[key] = g
        self._upload(ws, Plan.concat(plans))
        g.replay()
        return self._full_logits(ws.logits[:n]), ws.x[:n]

    def capture_decode_sample(self, b: int):
        """Capture decode + token selection for batch size ``b`` (reference: src/gpu.rs:3987-4081
        ``capture_decode_sample_graph``): backbone, then penalties / top-k / nucleus / draw from the parameter block the
        sampler uploaded for this step; the chosen ids land in ``sampler.out_tok``."""
        ws = self.ws
        self._upload(ws, Plan.decode([0] * b, [0] * b, list(range(b))))
        saved = [(t, t[:, :b].clone()) for t in (self.S, self.conv) if t is not None]
        kv = self._kv_tensors()
        saved += [(t, t[:, :b, :, :1].clone()) for t in kv]
        from ..engine.sampling import SamplingParams
        self.sampler.upload([SamplingParams()] * b, u=[0.5] * b)
        torch.cuda.synchronize(self.dev)
        s = torch.cuda.Stream(device=self.dev)
        s.wait_stream(torch.cuda.current_stream(self.dev))
        with torch.cuda.stream(s):
            for _ in range(2):
                self._backbone(ws, b, b, False, False, False)
                self.sampler.select(ws.logits, b, True)
        torch.cuda.current_stream(self.dev).wait_stream(s)
        torch.cuda.synchronize(self.dev)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._backbone(ws, b, b, False, False, False)
            self.sampler.select(ws.logits, b, True)
        for t, keep in saved:
            if any(t is x for x in kv):
                t[:, :b, :, :1].copy_(keep)
            else:
                t[:, :b].copy_(keep)
        self.graphs[("sample", b)] = g
        return g

    def ensure_sample_graph(self, b: int):
        """Capture the decode + sample graph for batch ``b`` if needed. Capturing stages placeholder sampling
        parameters, so call this before ``sampler.upload`` for the step."""
        if ("sample", b) not in self.graphs:
            self.capture_decode_sample(b)

    def replay_decode_sample(self, tokens, pos, slots) -> torch.Tensor:
        """Graph replay of decode + sampling; the caller has staged this step's sampling parameters with
        ``sampler.upload`` (after ``ensure_sample_graph``). Returns the device tensor of chosen ids."""
        b = len(tokens)
        self._upload(self.ws, Plan.decode(tokens, pos, slots))
        self.graphs[("sample", b)].replay()
        return self.sampler.out_tok[:b]

    def time_decode_steps(self, tok: int, pos: int, slot: int, steps: int) -> float:
        """Device time (ms) of ``steps`` consecutive batch-1 greedy decode steps with the sampled token fed
        back on the device: graph replays separated only by the tiny device-side updates of the step inputs."""
        ws = self.ws
        if ("decode", 1) not in self.graphs:
            self.capture_decode(1)
        g = self.graphs[("decode", 1)]
        self._upload(ws, Plan.decode([tok], [pos], [slot]))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        adv = ws.meta[1:6, :1]          # pos, kv_slot(unchanged, +0), kv_row, lens, base
        inc = torch.tensor([[1], [0], [1], [1], [1]], dtype=torch.int32, device=self.dev)
        torch.cuda.synchronize(self.dev)
        e0.record()
        for _ in range(steps):
            g.replay()
            ws.tok[:1].copy_(ws.out_tok[:1])
            adv.add_(inc)
        e1.record()
        torch.cuda.synchronize(self.dev)
        return e0.elapsed_time(e1)

    def replay_decode(self, tokens, pos, slots) -> torch.Tensor:
        """Graph replay of a greedy decode step; returns the device tensor of token ids."""
        b = len(tokens)
        g = self.graphs.get(("decode", b))
        if g is None:
            g = self.capture_decode(b)
        self._upload(self.ws, Plan.decode(tokens, pos, slots))
        g.replay()
        return self.ws.out_tok[:b]

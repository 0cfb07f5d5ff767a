"""Token selection on the GPU: penalties, top-k, nucleus, draw, and the stochastic speculative accept, for up to
``cap`` logits rows per call, over a full or a vocabulary-sharded LM head.

Every quantity the kernels need (sampling parameters, the uniforms of the request's keyed generator, penalty token
lists, draft tokens) is packed into one pinned host buffer and uploaded with a single copy; the kernels are
enqueue-only, so a decode step that samples can be captured in a CUDA graph, and a step costs one device->host read
(the chosen tokens, or the accept count and next token of a verify). Under tensor parallelism each rank reduces its
shard to the row's local top-64, the ranks exchange those 512-byte lists with the small peer-memory all-gather, and
every rank finishes the nucleus identically; full logits never travel (reference: kernels/gpu_batch.cu:2206-2272
``sample_b``, :2405 ``sample_prob_b``, :2483-2600 ``spec_verify_b``, src/gpu.rs:3717-3747 for the vocabulary merge it
replaces).
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence, Tuple

import torch

from ..ops import kernels as K
from ..ops import lib as _lib
from ..ops.lib import c_int, ptr, stream
from . import sampling as S

MAXK = S.MAX_TOPK
# rows of the packed parameter block ([row, cap] int32; float rows are bit-cast)
R_TEMP, R_TOPP, R_U, R_UACC, R_UVER, R_REP, R_PRES, R_FREQ, R_TOPK, R_NTOK, R_DRAFT, R_COL0, R_ND = range(13)
N_ROWS = 13


class DeviceSampler:
    def __init__(self, device, vocab_local: int, cap: int = 16, comm=None):
        self.dev = torch.device(device)
        self.cap, self.vl = cap, vocab_local
        self.comm = comm if (comm is not None and comm.world > 1) else None
        self.world = self.comm.world if self.comm else 1
        self.rank = self.comm.rank if self.comm else 0
        words = N_ROWS * cap + 2 * cap * S.MAX_PENALTY_TOKENS
        self.host = torch.zeros(words, dtype=torch.int32).pin_memory()
        self.devbuf = torch.zeros(words, dtype=torch.int32, device=self.dev)
        self.h_rows = self.host[:N_ROWS * cap].view(N_ROWS, cap)
        self.h_f = self.h_rows.view(torch.float32)
        self.h_toks = self.host[N_ROWS * cap:N_ROWS * cap + cap * 64].view(cap, 64)
        self.h_cnts = self.host[N_ROWS * cap + cap * 64:].view(cap, 64)
        # numpy views of the same pinned block: element writes through tensor indexing cost microseconds each, and a
        # step writes a dozen per lane
        self.h_rows, self.h_f = self.h_rows.numpy(), self.h_f.numpy()
        self.h_toks, self.h_cnts = self.h_toks.numpy(), self.h_cnts.numpy()
        d_rows = self.devbuf[:N_ROWS * cap].view(N_ROWS, cap)
        d_f = d_rows.view(torch.float32)
        self.temp, self.top_p, self.u, self.u_acc, self.u_ver = d_f[R_TEMP], d_f[R_TOPP], d_f[R_U], d_f[R_UACC], d_f[R_UVER]
        self.rep, self.pres, self.freq = d_f[R_REP], d_f[R_PRES], d_f[R_FREQ]
        self.top_k, self.n_toks, self.drafts = d_rows[R_TOPK], d_rows[R_NTOK], d_rows[R_DRAFT]
        self.col0, self.nd = d_rows[R_COL0], d_rows[R_ND]
        self.toks = self.devbuf[N_ROWS * cap:N_ROWS * cap + cap * 64].view(cap, 64)
        self.cnts = self.devbuf[N_ROWS * cap + cap * 64:].view(cap, 64)
        chunks = K.topk_chunks(vocab_local)
        self.cand_chunks = torch.zeros(cap * chunks * MAXK * 2, dtype=torch.float32, device=self.dev)
        self.cand = torch.zeros(cap * MAXK * 2, dtype=torch.float32, device=self.dev)
        self.gathered = torch.zeros(self.world * cap * MAXK * 2, dtype=torch.float32, device=self.dev) if self.comm else None
        self.out_tok = torch.zeros(cap, dtype=torch.int32, device=self.dev)
        self.ids = torch.zeros((cap, MAXK), dtype=torch.int32, device=self.dev)
        self.probs = torch.zeros((cap, MAXK), dtype=torch.float32, device=self.dev)
        self.keep = torch.zeros(cap, dtype=torch.int32, device=self.dev)
        self.result = torch.zeros((cap, 2), dtype=torch.int32, device=self.dev)
        self._uploaded = None

    # ------------------------------------------------------------ host side: pack + one copy
    def upload(self, params: Sequence[S.SamplingParams], u: Optional[Sequence[float]] = None,
               histories: Optional[Sequence[Sequence[int]]] = None, drafts: Optional[Sequence[int]] = None,
               u_acc: Optional[Sequence[float]] = None, u_ver: Optional[Sequence[float]] = None,
               lanes: Optional[Sequence[Tuple[int, int]]] = None) -> bool:
        """Stage the rows' parameters. ``histories[r]`` is the token history row r is penalised with; ``lanes`` is a
        list of (first column, number of drafts) for ``verify``. Returns True when any row has a penalty."""
        n = len(params)
        assert n <= self.cap, (n, self.cap)
        if self._uploaded is not None:
            self._uploaded.synchronize()              # the previous copy must have left the pinned block
        hf, hi = self.h_f, self.h_rows
        any_pen = False
        for r, p in enumerate(params):
            hf[R_TEMP, r], hf[R_TOPP, r] = p.temperature, p.top_p
            hf[R_U, r] = u[r] if u is not None else 0.0
            hf[R_UACC, r] = u_acc[r] if u_acc is not None else 0.0
            hf[R_UVER, r] = u_ver[r] if u_ver is not None else 0.0
            hf[R_REP, r], hf[R_PRES, r], hf[R_FREQ, r] = p.repetition_penalty, p.presence_penalty, p.frequency_penalty
            hi[R_TOPK, r] = int(p.top_k)
            hi[R_DRAFT, r] = int(drafts[r]) if drafts is not None and r < len(drafts) else -1
            nt = 0
            if histories is not None and p.has_penalty and histories[r]:
                toks, cnts = S.penalty_list(histories[r])
                nt = len(toks)
                self.h_toks[r, :nt] = toks
                self.h_cnts[r, :nt] = cnts
                any_pen = True
            hi[R_NTOK, r] = nt
        if lanes is not None:
            for l, (c0, nd) in enumerate(lanes):
                hi[R_COL0, l], hi[R_ND, l] = c0, nd
        self.devbuf.copy_(self.host, non_blocking=True)
        if self._uploaded is None:
            self._uploaded = torch.cuda.Event()
        self._uploaded.record()
        return any_pen

    # ------------------------------------------------------------ device side: enqueue only
    def select(self, logits: torch.Tensor, n: int, penalise: bool, want_nucleus: bool = False) -> torch.Tensor:
        """Rows ``logits[:n]`` (fp32, this rank's vocabulary shard; modified in place when penalised) -> chosen token per
        row in ``out_tok[:n]`` (greedy rows: arg-max, lowest index on ties). With ``want_nucleus`` the rows' nuclei
        (ids, probs, count) are left in ``ids`` / ``probs`` / ``keep`` for ``verify``."""
        assert logits.dtype == torch.float32 and logits.shape[1] == self.vl and n <= self.cap
        off = self.rank * self.vl
        if penalise:
            K.penalty_sharded(logits, n, self.toks, self.cnts, self.n_toks, self.rep, self.pres, self.freq, off)
        K.topk_local(logits, n, self.temp, self.top_k, off, self.cand_chunks, self.cand)
        if self.comm is not None:
            rc = self.comm.L.vg_comm_allgather_small(ctypes.byref(self.comm.ctx), ptr(self.cand), ptr(self.gathered),
                                                     c_int(n * MAXK * 8), stream())
            _lib.check(rc, "vg_comm_allgather_small")
            return self._finish_gathered(n, want_nucleus)
        K.nucleus_finish(self.cand, 1, MAXK, n, self.temp, self.top_k, self.top_p, self.u, self.out_tok,
                         self.ids if want_nucleus else None, self.probs if want_nucleus else None,
                         self.keep if want_nucleus else None)
        return self.out_tok[:n]

    def _finish_gathered(self, n: int, want_nucleus: bool) -> torch.Tensor:
        # the all-gather stores rank q's payload at q * (n * 64) pairs: regroup per row with one strided copy so
        # a row's `world` lists are contiguous, then merge
        g = self.gathered[:self.world * n * MAXK * 2].view(self.world, n, MAXK * 2)
        per_row = self._per_row(n)
        per_row.copy_(g.permute(1, 0, 2))
        K.nucleus_finish(per_row, self.world, self.world * MAXK, n, self.temp, self.top_k, self.top_p, self.u, self.out_tok,
                         self.ids if want_nucleus else None, self.probs if want_nucleus else None,
                         self.keep if want_nucleus else None)
        return self.out_tok[:n]

    def _per_row(self, n: int) -> torch.Tensor:
        buf = getattr(self, "_rowbuf", None)
        if buf is None:
            buf = self._rowbuf = torch.zeros(self.cap * self.world * MAXK * 2, dtype=torch.float32, device=self.dev)
        return buf[:n * self.world * MAXK * 2].view(n, self.world, MAXK * 2)

    def verify(self, n_lanes: int) -> torch.Tensor:
        """After ``select(..., want_nucleus=True)`` over all lanes' verify columns: (accepted drafts, next token) per
        lane in ``result[:n_lanes]``."""
        K.spec_verify(self.ids, self.probs, self.keep, self.drafts, self.u_acc, self.u_ver, self.col0, self.nd, n_lanes,
                      self.result)
        return self.result[:n_lanes]

    # ------------------------------------------------------------ conveniences (upload + enqueue + read back)
    def pick(self, logits: torch.Tensor, params: Sequence[S.SamplingParams], histories: Sequence[Sequence[int]],
             keys: Sequence[int]) -> List[int]:
        """One token per row, as ``Scheduler._pick_token`` on the host would choose it."""
        n = len(params)
        u = [S.rng_uniform(keys[i], S.DOMAIN_SAMPLE, 0) for i in range(n)]
        pen = self.upload(params, u=u, histories=histories)
        return self.select(logits, n, pen).tolist()

    def chain_accept(self, logits: torch.Tensor, p: S.SamplingParams, history: Sequence[int], drafts: Sequence[int],
                     key: int) -> Tuple[int, int]:
        """Stochastic accept of one lane's greedy draft chain: ``logits`` has len(drafts) + 1 rows; row t is penalised
        with the history extended by the first t drafts. Returns (accepted drafts, next token)."""
        n = len(drafts) + 1
        hist = list(history)
        hists = []
        for t in range(n):
            hists.append(list(hist))
            if t < len(drafts):
                hist.append(drafts[t])
        u_acc = [S.rng_uniform(key, S.DOMAIN_ACCEPT, t) for t in range(n)]
        u_ver = [S.rng_uniform(key, S.DOMAIN_VERIFY, t) for t in range(n)]
        pen = self.upload([p] * n, histories=hists, drafts=list(drafts), u_acc=u_acc, u_ver=u_ver, lanes=[(0, len(drafts))])
        self.select(logits, n, pen, want_nucleus=True)
        nacc, nxt = self.verify(1)[0].tolist()
        return int(nacc), int(nxt)

"""Thin Python wrappers over the non-GEMM kernels (norms, RoPE/KV write, attention, GatedDeltaNet,
embedding, sampling). Each wrapper validates shapes/dtypes, enqueues on the current stream and
returns the output tensor; none of them allocates unless the caller omits ``out``."""
from __future__ import annotations

from typing import Optional

import torch

from ..models.weights import QLinear
from . import lib as _lib
from .gemm import _FMT_CODE
from .lib import c_float, c_int, c_ll, ptr, stream


def add_rmsnorm(res: torch.Tensor, delta: Optional[torch.Tensor], w: torch.Tensor, eps: float, n: int,
                out16: Optional[torch.Tensor] = None, out_bf: Optional[torch.Tensor] = None, plus_one: bool = True):
    """``res[:n] += delta[:n]`` (when delta is given), then RMSNorm of the updated rows into ``out16``
    (f16) and/or ``out_bf`` (bf16). ``res`` is bf16 [rows, h] and is updated in place."""
    h = res.shape[1]
    assert res.dtype == torch.bfloat16 and w.dtype == torch.float32
    rc = _lib.lib().vg_add_rmsnorm(ptr(res), ptr(delta), ptr(w), ptr(out16), ptr(out_bf), c_int(n), c_int(h),
                                   c_float(eps), c_int(1 if plus_one else 0), c_int(res.stride(0)),
                                   c_int(delta.stride(0) if delta is not None else 0), stream())
    _lib.check(rc, "vg_add_rmsnorm")


def attn_prep(qkv, q_norm, k_norm, pos, slot, kv_row, q_out, kc, vc, n, nh, nkv, hd, rdim, eps, theta, gated=True,
              k_scale=None, v_scale=None):
    """q/k norm + partial RoPE + cache write. With ``k_scale`` / ``v_scale`` the cache is 4-bit: ``kc`` / ``vc`` hold
    code bytes ``[slots, nkv, max_seq, hd/2]`` and the scales are f16 ``[slots, nkv, max_seq, hd/16]``."""
    max_seq = kc.shape[2]
    rc = _lib.lib().vg_attn_prep(ptr(qkv), c_int(qkv.stride(0)), ptr(q_norm), ptr(k_norm), ptr(pos), ptr(slot),
                                 ptr(kv_row), ptr(q_out), ptr(kc), ptr(vc), c_int(n), c_int(nh), c_int(nkv), c_int(hd),
                                 c_int(rdim), c_int(max_seq), c_float(eps), c_float(theta), c_int(1 if gated else 0),
                                 ptr(k_scale), ptr(v_scale), stream())
    _lib.check(rc, "vg_attn_prep")


def swiglu(gu: torch.Tensor, out16: torch.Tensor, n: int, inter: int):
    rc = _lib.lib().vg_swiglu(ptr(gu), ptr(out16), c_int(n), c_int(inter), c_int(gu.stride(0)), stream())
    _lib.check(rc, "vg_swiglu")


def cast_f16(x: torch.Tensor, out16: Optional[torch.Tensor] = None) -> torch.Tensor:
    assert x.is_contiguous() and x.dtype in (torch.float32, torch.bfloat16)
    if out16 is None:
        out16 = torch.empty(x.shape, dtype=torch.float16, device=x.device)
    rc = _lib.lib().vg_cast_f16(ptr(x), c_int(1 if x.dtype == torch.float32 else 0), ptr(out16), c_ll(x.numel()), stream())
    _lib.check(rc, "vg_cast_f16")
    return out16


def embed_gather(e: QLinear, tok: torch.Tensor, out: torch.Tensor, n: int):
    if e.fmt == "nvfp4":
        table, sc = e.packed, e.scales
    elif e.fmt == "fp8":
        table, sc = e.codes, None
    else:
        table, sc = e.w, None
    rc = _lib.lib().vg_embed_gather(ptr(table), ptr(sc), ptr(e.row_scale), ptr(tok), ptr(out), c_int(n), c_int(e.k),
                                    c_int(_FMT_CODE[e.fmt]), stream())
    _lib.check(rc, "vg_embed_gather")


def attn_scratch_floats(n: int, nh: int, hd: int, ns_grid: int = 32) -> int:
    return int(_lib.lib().vg_attn_scratch_floats(c_int(n), c_int(nh), c_int(hd), c_int(ns_grid)))


def attn_decode(q, kc, vc, lens, slots, part, out16, n, nh, nkv, hd, gate=None, base=None, path=None,
                ns_grid: int = 32, direct: bool = False, k_scale=None, v_scale=None):
    """Split-K GQA attention of ``n`` columns over the slotted cache. ``lens[c]`` keys are attended by
    column c; ``part`` is the fp32 partial buffer (scratch, ``attn_scratch_floats`` elements). With
    ``k_scale`` / ``v_scale`` the cache is 4-bit (see ``attn_prep``)."""
    max_seq = kc.shape[2]
    if k_scale is not None:
        rc = _lib.lib().vg_attn_decode_q4(ptr(q), ptr(kc), ptr(vc), ptr(k_scale), ptr(v_scale), ptr(lens), ptr(slots),
                                          ptr(base), ptr(path), c_int(path.stride(0) if path is not None else 0), ptr(part),
                                          c_int(n), c_int(nh), c_int(nkv), c_int(hd), c_int(max_seq), c_int(ns_grid),
                                          c_int(1 if direct else 0), ptr(gate),
                                          c_int(gate.stride(0) if gate is not None else 0), ptr(out16), stream())
        _lib.check(rc, "vg_attn_decode_q4", 1 if direct else 2)
        return
    rc = _lib.lib().vg_attn_decode(ptr(q), ptr(kc), ptr(vc), ptr(lens), ptr(slots), ptr(base), ptr(path),
                                   c_int(path.stride(0) if path is not None else 0), ptr(part), c_int(n), c_int(nh),
                                   c_int(nkv), c_int(hd), c_int(max_seq), c_int(ns_grid), c_int(1 if direct else 0),
                                   ptr(gate), c_int(gate.stride(0) if gate is not None else 0), ptr(out16), stream())
    _lib.check(rc, "vg_attn_decode", 1 if direct else 2)


def attn_prefill_tc(q, kc, vc, vT, slot: int, pos0: int, n: int, nh: int, nkv: int, hd: int, out16, gate=None,
                    k_scale=None, v_scale=None, k_rows=None):
    """Causal prefill attention on the tensor cores for one lane: queries ``q[:n]`` (bf16 ``[cap, nh*hd]``) at
    positions ``pos0 ..``, keys / values = the lane's cache rows ``[0, pos0 + n)``. ``vT`` is the transposed-value
    scratch ``[nkv, hd, cap_keys]`` this call refreshes first. A 4-bit cache (``k_scale`` / ``v_scale``) is first
    expanded to bf16: keys into ``k_rows`` ``[1, nkv, max_seq, hd]``, values straight into ``vT``."""
    max_seq = kc.shape[2]
    L = _lib.lib()
    if k_scale is not None:
        rc = L.vg_kv_q4_dequant(ptr(kc), ptr(k_scale), c_int(slot), c_int(nkv), c_int(hd), c_int(max_seq), c_int(pos0 + n),
                                ptr(k_rows), ptr(None), c_int(0), stream())
        _lib.check(rc, "vg_kv_q4_dequant")
        rc = L.vg_kv_q4_dequant(ptr(vc), ptr(v_scale), c_int(slot), c_int(nkv), c_int(hd), c_int(max_seq), c_int(pos0 + n),
                                ptr(None), ptr(vT), c_int(vT.shape[2]), stream())
        _lib.check(rc, "vg_kv_q4_dequant")
        kc, slot = k_rows, 0
    else:
        rc = L.vg_attn_transpose_v(ptr(vc), ptr(vT), c_int(slot), c_int(nkv), c_int(hd), c_int(max_seq), c_int(pos0 + n),
                                   c_int(vT.shape[2]), stream())
        _lib.check(rc, "vg_attn_transpose_v")
    rc = L.vg_attn_prefill_tc(ptr(q), c_int(q.shape[0]), ptr(kc), ptr(vT), c_int(vT.shape[2]), c_int(slot), c_int(nkv),
                              c_int(nh), c_int(hd), c_int(max_seq), c_int(pos0), c_int(n), c_float(hd ** -0.5),
                              ptr(gate), c_int(gate.stride(0) if gate is not None else 0), ptr(out16),
                              ptr(_lib.err_word(q.device)), stream())
    _lib.check(rc, "vg_attn_prefill_tc")


def gdn_conv(x, state, w, in_slot, parent, out_slot, out, n, conv_dim, ck, phase: int = 3):
    rc = _lib.lib().vg_gdn_conv(ptr(x), c_int(x.stride(0)), ptr(state), ptr(w), ptr(in_slot), ptr(parent),
                                ptr(out_slot), ptr(out), c_int(n), c_int(conv_dim), c_int(ck), c_int(phase), stream())
    _lib.check(rc, "vg_gdn_conv")


def gdn_conv_chain(x, state, w, in_slot, parent, out_slot, out, n, conv_dim, ck) -> bool:
    """Conv + SiLU + state update of one linear chain (prefill); False when the shape is not covered (the caller
    then runs the generic two-phase form)."""
    if ck != 4 or conv_dim % 8 or x.stride(0) % 8:
        return False
    rc = _lib.lib().vg_gdn_conv_chain(ptr(x), c_int(x.stride(0)), ptr(state), ptr(w), ptr(in_slot), ptr(parent),
                                      ptr(out_slot), ptr(out), c_int(n), c_int(conv_dim), c_int(ck), stream())
    _lib.check(rc, "vg_gdn_conv_chain")
    return True


def gdn_step(qkv, proj, off_z, off_b, off_a, S, A_log, dt_bias, norm_w, chain_start, chain_len, n_chains,
             in_slot, parent, out_slot, out16, nk, nv, kd, vd, eps, quant=None):
    """``quant = (bq, sfb, g0, col_ctr)`` makes the kernel also emit every output row as the FP4 activation
    series (the head that finishes a column last quantises it); ``col_ctr`` is 48 zeroed int32 words."""
    bq, sfb, g0, ctr = quant if quant is not None else (None, None, None, None)
    assert ctr is None or ctr.numel() >= 48
    rc = _lib.lib().vg_gdn_step(ptr(qkv), ptr(proj), c_int(proj.stride(0)), c_int(off_z), c_int(off_b), c_int(off_a),
                                ptr(S), ptr(A_log), ptr(dt_bias), ptr(norm_w), ptr(chain_start), ptr(chain_len),
                                c_int(n_chains), ptr(in_slot), ptr(parent), ptr(out_slot), ptr(out16), c_int(nk),
                                c_int(nv), c_int(kd), c_int(vd), c_float(eps), ptr(bq),
                                c_int(bq.stride(0) if bq is not None else 0), ptr(sfb), ptr(g0), ptr(ctr),
                                ptr(_lib.err_word(qkv.device)), stream())
    _lib.check(rc, "vg_gdn_step")


def gdn_prefill(qkv, proj, off_z, off_b, off_a, S, A_log, dt_bias, norm_w, t0, tn, in_slot, out_slot, out16, nk, nv, kd, vd,
                eps, o_scratch=None, split: int = 0):
    """One linear chain of ``tn`` columns (prefill): bit-identical to ``gdn_step`` on that chain, with the
    per-token reductions batched so the critical path is the thread-local recurrence. With ``o_scratch``
    (fp32, ``(t0 + tn) * nv * vd`` elements) each head is split over ``split`` CTAs (0 = automatic) and the
    gated output norm runs as a second kernel."""
    rc = _lib.lib().vg_gdn_prefill(ptr(qkv), ptr(proj), c_int(proj.stride(0)), c_int(off_z), c_int(off_b), c_int(off_a),
                                   ptr(S), ptr(A_log), ptr(dt_bias), ptr(norm_w), c_int(t0), c_int(tn), ptr(in_slot),
                                   ptr(out_slot), ptr(out16), c_int(nk), c_int(nv), c_int(kd), c_int(vd), c_float(eps),
                                   ptr(o_scratch), c_int(split), stream())
    _lib.check(rc, "vg_gdn_prefill", 2 if o_scratch is not None else 1)


def argmax(logits: torch.Tensor, n: int, out: torch.Tensor, out_val: Optional[torch.Tensor] = None,
           idx_offset: int = 0):
    assert logits.dtype == torch.float32
    rc = _lib.lib().vg_argmax(ptr(logits), c_int(n), c_int(logits.shape[1]), c_int(logits.stride(0)), ptr(out),
                              ptr(out_val), c_int(idx_offset), stream())
    _lib.check(rc, "vg_argmax")


def penalty(logits, n, toks, counts, n_toks, rep, pres, freq):
    """In-place repetition / presence / frequency penalties: row r's tokens ``toks[r, :n_toks[r]]`` with ``counts``."""
    penalty_sharded(logits, n, toks, counts, n_toks, rep, pres, freq, 0)


def nucleus(logits, n, temp, top_k, top_p, seed, out_tok=None, ids=None, probs=None, n_keep=None):
    rc = _lib.lib().vg_nucleus(ptr(logits), c_int(n), c_int(logits.shape[1]), c_int(logits.stride(0)), ptr(temp),
                               ptr(top_k), ptr(top_p), ptr(seed), ptr(out_tok), ptr(ids), ptr(probs), ptr(n_keep),
                               stream())
    _lib.check(rc, "vg_nucleus")


def nll(logits, n, target, out):
    rc = _lib.lib().vg_nll(ptr(logits), c_int(n), c_int(logits.shape[1]), c_int(logits.stride(0)), ptr(target),
                           ptr(out), stream())
    _lib.check(rc, "vg_nll")


def penalty_sharded(logits, n, toks, counts, n_toks, rep, pres, freq, idx_offset: int = 0):
    """``penalty`` over a vocabulary shard: token ids are global, ``idx_offset`` is the shard's first id."""
    rc = _lib.lib().vg_penalty(ptr(logits), c_int(n), c_int(logits.shape[1]), c_int(logits.stride(0)), ptr(toks),
                               ptr(counts), ptr(n_toks), c_int(toks.shape[1]), ptr(rep), ptr(pres), ptr(freq),
                               c_int(idx_offset), stream())
    _lib.check(rc, "vg_penalty")


def topk_chunks(v: int) -> int:
    return int(_lib.lib().vg_topk_chunks(c_int(v)))


def topk_local(logits, n, temp, top_k, idx_offset, cand_chunks, out_cand):
    """Per-row top-K (K = clamp(top_k, 1, 64); 1 for greedy rows) as (value, global index) pairs in selection order."""
    rc = _lib.lib().vg_topk_local(ptr(logits), c_int(n), c_int(logits.shape[1]), c_int(logits.stride(0)), ptr(temp),
                                  ptr(top_k), c_int(idx_offset), ptr(cand_chunks), ptr(out_cand), stream())
    _lib.check(rc, "vg_topk_local", 2)


def nucleus_finish(lists, n_lists, row_stride_pairs, n, temp, top_k, top_p, u, out_tok=None, ids=None, probs=None,
                   n_keep=None):
    rc = _lib.lib().vg_nucleus_finish(ptr(lists), c_int(n_lists), c_int(row_stride_pairs), c_int(n), ptr(temp), ptr(top_k),
                                      ptr(top_p), ptr(u), ptr(out_tok), ptr(ids), ptr(probs), ptr(n_keep), stream())
    _lib.check(rc, "vg_nucleus_finish")


def spec_verify(ids, probs, n_keep, drafts, u_acc, u_ver, col0, nd, n_lanes, result):
    rc = _lib.lib().vg_spec_verify(ptr(ids), ptr(probs), ptr(n_keep), ptr(drafts), ptr(u_acc), ptr(u_ver), ptr(col0),
                                   ptr(nd), c_int(n_lanes), ptr(result), stream())
    _lib.check(rc, "vg_spec_verify")


def gdn_chunk_work_bytes(tn: int, nv: int) -> int:
    return int(_lib.lib().vg_gdn_chunk_work_bytes(c_int(tn), c_int(nv)))


def gdn_chunk_prefill(qkv, proj, off_z, off_b, off_a, S, A_log, dt_bias, norm_w, t0, tn, in_slot, out_slot, out16, nk, nv, kd,
                      vd, eps, work, o_raw):
    """One linear chain of ``tn`` columns in chunked form on the tensor cores (64-token chunks, tf32 MMAs, fp32 state):
    agrees with ``gdn_prefill`` / ``gdn_step`` to tf32 rounding. The carried state comes from slot ``in_slot[t0]`` and
    is written to ``out_slot[t0 + tn - 1]`` when that is >= 0; there are no other checkpoints inside a call. ``work``:
    uint8 scratch of ``gdn_chunk_work_bytes(tn, nv)`` bytes, 1024-byte aligned; ``o_raw``: fp32, ``(t0 + tn) * nv * vd``."""
    L = _lib.lib()
    L.vg_gdn_chunk_work_bytes.restype = c_ll
    assert work.data_ptr() % 1024 == 0 and work.numel() >= gdn_chunk_work_bytes(tn, nv)
    assert o_raw.numel() >= (t0 + tn) * nv * vd and qkv.is_contiguous()
    rc = L.vg_gdn_chunk_prefill(ptr(qkv), ptr(proj), c_int(proj.stride(0)), c_int(off_z), c_int(off_b), c_int(off_a), ptr(S),
                                ptr(A_log), ptr(dt_bias), ptr(norm_w), c_int(t0), c_int(tn), ptr(in_slot), ptr(out_slot),
                                ptr(out16), c_int(nk), c_int(nv), c_int(kd), c_int(vd), c_float(eps), ptr(work), ptr(o_raw),
                                ptr(_lib.err_word(qkv.device)), stream())
    _lib.check(rc, "vg_gdn_chunk_prefill", 3)


def attn_decode_tc(q, kc, vc, lens, slots, part, out16, n, nh, nkv, hd, gate=None, ns_grid: int = 32, block_table=None):
    """Tensor-core split-K decode attention (head_dim 256, bf16 cache, query group <= 16). Slotted cache
    ``[slots, nkv, max_seq, hd]``, or with ``block_table`` (int32 ``[n, pages]``) a pool ``[pages, nkv, 128, hd]`` of
    128-key pages; column c's keys ``[128 p, 128 p + 128)`` live in page ``block_table[c, p]``."""
    assert kc.dtype == torch.bfloat16 and kc.is_contiguous() and vc.is_contiguous() and hd == 256
    rows = kc.numel() // hd
    max_seq = kc.shape[2]
    rc = _lib.lib().vg_attn_decode_tc(ptr(q), ptr(kc), ptr(vc), c_ll(rows), ptr(lens), ptr(slots), ptr(block_table),
                                      c_int(block_table.stride(0) if block_table is not None else 0), ptr(part), c_int(n),
                                      c_int(nh), c_int(nkv), c_int(hd), c_int(max_seq), c_int(ns_grid), ptr(gate),
                                      c_int(gate.stride(0) if gate is not None else 0), ptr(out16),
                                      ptr(_lib.err_word(q.device)), stream())
    _lib.check(rc, "vg_attn_decode_tc", 2)

"""Linear layers on the GPU: weight re-tiling for the tensor-core GEMM and the call wrappers.

``prepare`` turns a canonical ``QLinear`` into the tile-major layout ``gemm_tc.cu`` streams with 1-D
bulk copies: ``[M/128][K/128]`` tiles of 128 rows x 128 k, each tile contiguous, with the 16-byte
chunks of a row pre-swizzled so the dequantising warps read shared memory without bank conflicts.
This load-time transform is the counterpart of the reference's MMA-fragment repack
(reference: src/quant.rs:424-537); it is internal to the engine and not part of the file format.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import ctypes

import torch

from ..models.weights import QLinear
from . import lib as _lib
from .lib import c_float, c_int, c_void_p, ptr, stream

WF_NVFP4, WF_FP8, WF_F16, WF_BF16 = 0, 1, 2, 3
_FMT_CODE = {"nvfp4": WF_NVFP4, "fp8": WF_FP8, "bf16": WF_BF16}


@dataclass
class TcWeight:
    wt: torch.Tensor               # uint8, tile-major
    row_scale: Optional[torch.Tensor]
    m: int
    k: int
    fmt: int
    splitk: int


def _pad2(t: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    if t.shape[0] == rows and t.shape[1] == cols:
        return t
    out = torch.zeros((rows, cols), dtype=t.dtype, device=t.device)
    out[:t.shape[0], :t.shape[1]] = t
    return out


def _swizzle_chunks(t: torch.Tensor, fn) -> torch.Tensor:
    """t [..., 128 rows, C chunks, B bytes]: physical chunk c of row r takes logical chunk c ^ fn(r)."""
    C = t.shape[-2]
    r = torch.arange(128, device=t.device)
    idx = torch.arange(C, device=t.device)[None, :] ^ fn(r)[:, None]          # [128, C]
    idx = idx.reshape((1,) * (t.dim() - 3) + (128, C, 1)).expand(t.shape)
    return torch.gather(t, -2, idx)


def tile_nvfp4(packed: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    m, kh = packed.shape
    k = kh * 2
    mt, ks = (m + 127) // 128, (k + 127) // 128
    p = _pad2(packed, mt * 128, ks * 64).view(mt, 128, ks, 4, 16).permute(0, 2, 1, 3, 4)
    p = _swizzle_chunks(p, lambda r: (r >> 1) & 3).reshape(mt, ks, 8192)
    s = _pad2(scales, mt * 128, ks * 8).view(mt, 128, ks, 8).permute(0, 2, 1, 3).reshape(mt, ks, 1024)
    return torch.cat([p, s], dim=-1).contiguous()


def tile_fp8(codes: torch.Tensor) -> torch.Tensor:
    m, k = codes.shape
    mt, ks = (m + 127) // 128, (k + 127) // 128
    p = _pad2(codes, mt * 128, ks * 128).view(mt, 128, ks, 8, 16).permute(0, 2, 1, 3, 4)
    return _swizzle_chunks(p, lambda r: r & 7).reshape(mt, ks, 16384).contiguous()


def tile_f16(w: torch.Tensor) -> torch.Tensor:
    """bf16/f32 weights -> f16 UMMA tiles: per (m-tile, k-slab) two [128 x 64] K-major sub-tiles with
    the 128-byte swizzle already applied."""
    m, k = w.shape
    mt, ks = (m + 127) // 128, (k + 127) // 128
    h = _pad2(w.to(torch.float16), mt * 128, ks * 128).view(mt, 128, ks, 2, 8, 8).permute(0, 2, 3, 1, 4, 5)
    h = h.contiguous().view(torch.uint8).reshape(mt, ks, 2, 128, 8, 16)
    return _swizzle_chunks(h, lambda r: r & 7).reshape(mt, ks, 32768).contiguous()


_resident = {}


def _resident_ctas(fmt: int) -> int:
    if fmt not in _resident:
        _resident[fmt] = max(1, int(_lib.lib().vg_gemm_tc_resident_ctas(c_int(fmt))))
    return _resident[fmt]


def choose_splitk(m: int, k: int, fmt: int) -> int:
    """Split-K factor for the decode shape: a pure function of (M, K, format), never of the batch
    width, so that every width <= 16 runs the same reduction tree."""
    tiles = (m + 127) // 128
    ks = (k + 127) // 128
    slots = _resident_ctas(fmt)
    # fill the resident CTA slots of one wave (two CTAs per SM for the NVFP4 decode tile), at most 6-way
    # (wider clusters schedule poorly), keeping at least 4 slabs of K per CTA
    return max(1, min(6, slots // max(tiles, 1), ks // 4))


def prepare(q: QLinear, keep_canonical: bool = True, splitk: Optional[int] = None) -> TcWeight:
    """Build (once) the tensor-core layout of a linear that lives on a CUDA device."""
    if q.kernel is not None:
        return q.kernel
    if q.fmt == "nvfp4":
        wt, fmt, rs = tile_nvfp4(q.packed, q.scales), WF_NVFP4, q.row_scale
    elif q.fmt == "fp8":
        wt, fmt, rs = tile_fp8(q.codes), WF_FP8, q.row_scale
    else:
        wt, fmt, rs = tile_f16(q.w), WF_F16, None
    mt = (q.m + 127) // 128
    if rs is not None and rs.numel() < mt * 128:
        rs = torch.cat([rs, torch.zeros(mt * 128 - rs.numel(), dtype=rs.dtype, device=rs.device)])
    sk = splitk if splitk is not None else choose_splitk(q.m, q.k, fmt)
    q.kernel = TcWeight(wt, rs, q.m, q.k, fmt, sk)
    if not keep_canonical:
        q.packed = q.scales = q.codes = q.w = None
    return q.kernel


def linear(q: QLinear, x16: torch.Tensor, n: Optional[int] = None, out: Optional[torch.Tensor] = None,
           out_f32: bool = False, comm=None, rs_rows: int = 0, ag: bool = False) -> torch.Tensor:
    """``out[n, m] = sum_k W[m, k] x[n, k]`` on the tensor cores. ``x16`` is f16 ``[rows >= n, K]``.
    With ``comm`` (a ``TpComm``) the epilogue also sums the result over the tensor-parallel ranks (decode widths).
    With ``comm`` and ``rs_rows`` (prefill widths) the epilogue instead pushes every partial tile to the rank that
    owns its token rows (``rs_rows`` per rank) and writes nothing to ``out``; ``comm.gemm_rs_finish`` completes it.
    With ``comm`` and ``ag`` the input is the all-gather landing zone (see ``TpComm.ag_gemm``)."""
    tw = prepare(q)
    assert x16.dtype == torch.float16 and x16.stride(1) == 1 and x16.shape[1] == tw.k
    n = x16.shape[0] if n is None else n
    if out is None:
        out = torch.empty((n, tw.m), dtype=torch.float32 if out_f32 else torch.bfloat16, device=x16.device)
    L = _lib.lib()
    rc = L.vg_gemm_tc(ptr(tw.wt), ptr(tw.row_scale), ptr(x16), c_int(x16.shape[0]), c_int(x16.stride(0)), ptr(out),
                      c_int(1 if out.dtype == torch.float32 else 0), c_int(tw.m), c_int(tw.k), c_int(n),
                      c_int(out.stride(0)), c_int(tw.fmt), c_int(1 if (rs_rows or ag) else tw.splitk),
                      ptr(_lib.err_word(x16.device)), ctypes.byref(comm.ctx) if comm is not None else c_void_p(0),
                      c_int(rs_rows), c_int(1 if ag else 0), stream())
    _lib.check(rc, "vg_gemm_tc")
    return out


def linear_simt(q: QLinear, x16: torch.Tensor, n: Optional[int] = None, out: Optional[torch.Tensor] = None,
                out_f32: bool = False) -> torch.Tensor:
    """Same contract as ``linear`` on CUDA cores over the canonical layout (small matrices, cross-checks)."""
    n = x16.shape[0] if n is None else n
    if out is None:
        out = torch.empty((n, q.m), dtype=torch.float32 if out_f32 else torch.bfloat16, device=x16.device)
    if q.fmt == "nvfp4":
        w, sc = q.packed, q.scales
    elif q.fmt == "fp8":
        w, sc = q.codes, None
    else:
        w, sc = q.w, None
    if w is None:
        raise _lib.KernelError("canonical weights were released; use linear()")
    L = _lib.lib()
    rc = L.vg_gemm_simt(ptr(w), ptr(sc), ptr(q.row_scale), ptr(x16), ptr(out),
                        c_int(1 if out.dtype == torch.float32 else 0), c_int(q.m), c_int(q.k), c_int(n),
                        c_int(x16.stride(0)), c_int(out.stride(0)), c_int(_FMT_CODE[q.fmt]), stream())
    _lib.check(rc, "vg_gemm_simt")
    return out


# ------------------------------------------------------------------ block-scaled FP4 path (N <= 16)

@dataclass
class Fp4Weight:
    wt: torch.Tensor               # uint8 [MT][K/256][16384 packed (128B-swizzled rows) + 2048 scale chunks]
    row_scale: Optional[torch.Tensor]
    m: int
    k: int
    kp: int                        # K padded to a multiple of 256
    splitk: int


def tile_nvfp4_mma(packed: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """Canonical NVFP4 -> the layout the FP4 tensor-core kernel consumes without any dequantisation:
    per (128-row tile, 256-k slab) the packed rows as a K-major UMMA tile with the 128-byte swizzle, followed
    by the block scales as four scale-factor chunks (one per K=64 step) in ``[row % 32][row // 32][k-block]``
    byte order, the order tcgen05.cp expects."""
    m, kh = packed.shape
    k = kh * 2
    mt, ksq = (m + 127) // 128, (k + 255) // 256
    p = _pad2(packed, mt * 128, ksq * 128).view(mt, 128, ksq, 8, 16).permute(0, 2, 1, 3, 4)
    p = _swizzle_chunks(p, lambda r: r & 7).reshape(mt, ksq, 16384)
    s = _pad2(scales, mt * 128, ksq * 16).view(mt, 4, 32, ksq, 4, 4)          # [mt, r1, r0, slab, step, kb]
    s = s.permute(0, 3, 4, 2, 1, 5).reshape(mt, ksq, 2048)                      # [mt, slab, step, r0, r1, kb]
    return torch.cat([p, s], dim=-1).contiguous()


def prepare_fp4(q: QLinear, splitk: Optional[int] = None) -> Fp4Weight:
    k4 = getattr(q, "kernel4", None)
    if k4 is not None:
        return k4
    assert q.fmt == "nvfp4" and q.packed is not None
    wt = tile_nvfp4_mma(q.packed, q.scales)
    mt = (q.m + 127) // 128
    rs = q.row_scale
    if rs.numel() < mt * 128:
        rs = torch.cat([rs, torch.zeros(mt * 128 - rs.numel(), dtype=rs.dtype, device=rs.device)])
    kp = ((q.k + 255) // 256) * 256
    if splitk is None:
        # one CTA per SM: never more CTAs than SMs, and at least eight 256-deep slabs per CTA (measured:
        # a second wave or a shorter K loop costs more than the extra parallelism returns)
        tiles, ks = mt, kp // 256
        sms = max(1, _resident_ctas(WF_NVFP4) // 2)
        splitk = max(1, min(8, sms // max(tiles, 1), ks // 8))
    q.kernel4 = Fp4Weight(wt, rs, q.m, q.k, kp, splitk)
    return q.kernel4


_fp4_act = {}


def fp4_buffers(dev, kp: int, rows: int = 16, tag: str = ""):
    """FP4 activation buffers (terms, scale chunks, per-row global scales) for inputs padded to ``kp``. Rows are
    grouped sixteen to a 64-row B tile. Buffers are shared by (device, kp, rows, tag): producers that may run
    concurrently (a second stream) use their own ``tag``."""
    tiles = (max(rows, 1) + 15) // 16
    key = (str(dev), kp, tiles, tag)
    b = _fp4_act.get(key)
    if b is None:
        b = (torch.zeros((64 * tiles, kp // 2), dtype=torch.uint8, device=dev),
             torch.zeros((tiles * (kp // 256), 2048), dtype=torch.uint8, device=dev),
             torch.zeros(16 * tiles, dtype=torch.float32, device=dev))
        _fp4_act[key] = b
    return b


def quantize_act_fp4(x16: torch.Tensor, n: int, kp: int):
    """Expand ``n <= 16`` f16 rows into the four-term NVFP4 series the FP4 GEMM consumes."""
    bq, sfb, g0 = fp4_buffers(x16.device, kp)
    rc = _lib.lib().vg_act_quant_fp4(ptr(x16), c_int(x16.stride(0)), c_int(n), c_int(x16.shape[1]), ptr(bq),
                                     c_int(bq.stride(0)), ptr(sfb), ptr(g0), stream())
    _lib.check(rc, "vg_act_quant_fp4")
    return bq, sfb, g0


def swiglu_fp4(gu: torch.Tensor, n: int, inter: int, out16: Optional[torch.Tensor] = None, bufs=None):
    """SwiGLU of ``gu[:n] = [gate | up]`` (bf16) emitted directly as the FP4 series for the down projection.
    ``bufs`` overrides the shared buffers (more than 16 rows, or a producer on another stream)."""
    kp = ((inter + 255) // 256) * 256
    bq, sfb, g0 = bufs if bufs is not None else fp4_buffers(gu.device, kp)
    assert bq.shape[0] >= 64 * ((n + 15) // 16) and bq.shape[1] * 2 == kp
    rc = _lib.lib().vg_swiglu_fp4(ptr(gu), c_int(gu.stride(0)), c_int(n), c_int(inter), ptr(bq), c_int(bq.stride(0)),
                                  ptr(sfb), ptr(g0), ptr(out16) if out16 is not None else c_void_p(0), stream())
    _lib.check(rc, "vg_swiglu_fp4")
    return bq, sfb, g0


def add_rmsnorm_fp4_ar(res: torch.Tensor, w: torch.Tensor, eps: float, n: int, comm, out16: Optional[torch.Tensor] = None,
                       plus_one: bool = True, mode: int = 1):
    """``add_rmsnorm_fp4`` whose delta is the tensor-parallel sum of the partial rows the preceding
    ``linear_fp4(..., push_only=True)`` of every rank published: ``mode`` 1 = (value, epoch) pairs in this rank's
    receive slots, 2 = fp32 rows in every rank's multimem slot, summed inside the NVLink switch."""
    h = res.shape[1]
    kp = ((h + 255) // 256) * 256
    bq, sfb, g0 = fp4_buffers(res.device, kp)
    rc = _lib.lib().vg_add_rmsnorm_fp4_ar(ptr(res), ptr(w), c_int(n), c_int(h), c_float(eps), c_int(1 if plus_one else 0),
                                          c_int(res.stride(0)), ptr(bq), c_int(bq.stride(0)), ptr(sfb), ptr(g0),
                                          ptr(out16) if out16 is not None else c_void_p(0), ctypes.byref(comm.ctx),
                                          c_int(mode), stream())
    _lib.check(rc, "vg_add_rmsnorm_fp4_ar")
    return bq, sfb, g0


def add_rmsnorm_fp4(res: torch.Tensor, delta: Optional[torch.Tensor], w: torch.Tensor, eps: float, n: int,
                    out16: Optional[torch.Tensor] = None, plus_one: bool = True):
    """``res += delta``; RMSNorm; the normalised rows leave as the FP4 series (and as f16 when ``out16`` is
    given, for consumers that are not on the FP4 path)."""
    h = res.shape[1]
    kp = ((h + 255) // 256) * 256
    bq, sfb, g0 = fp4_buffers(res.device, kp)
    rc = _lib.lib().vg_add_rmsnorm_fp4(ptr(res), ptr(delta) if delta is not None else c_void_p(0), ptr(w), c_int(n),
                                       c_int(h), c_float(eps), c_int(1 if plus_one else 0), c_int(res.stride(0)),
                                       c_int(delta.stride(0) if delta is not None else 0), ptr(bq), c_int(bq.stride(0)),
                                       ptr(sfb), ptr(g0), ptr(out16) if out16 is not None else c_void_p(0), stream())
    _lib.check(rc, "vg_add_rmsnorm_fp4")
    return bq, sfb, g0


class ConvEpi(ctypes.Structure):
    """Mirror of ``VgConvEpi``: the depthwise causal conv the GEMM epilogue runs on its conv-channel rows."""
    _fields_ = [("state", c_void_p), ("w", c_void_p), ("in_slot", c_void_p), ("parent", c_void_p),
                ("out_slot", c_void_p), ("out", c_void_p), ("conv_dim", c_int), ("ck", c_int)]

    @staticmethod
    def make(state, w, in_slot, parent, out_slot, out, conv_dim: int, ck: int) -> "ConvEpi":
        assert state.dtype == torch.float32 and w.dtype == torch.float32 and out.dtype == torch.float32
        assert out.is_contiguous() and state.is_contiguous()       # `out` is addressed as [n][conv_dim]
        return ConvEpi(state.data_ptr(), w.data_ptr(), in_slot.data_ptr(), parent.data_ptr(), out_slot.data_ptr(),
                       out.data_ptr(), conv_dim, ck)


def linear_fp4(q: QLinear, x16: torch.Tensor, n: int, out: Optional[torch.Tensor] = None, out_f32: bool = False,
               comm=None, act=None, conv: Optional[ConvEpi] = None, push_only: bool = False) -> torch.Tensor:
    """Decode-width linear on the block-scaled FP4 tensor-core path. ``act`` may carry an already quantised
    activation (several linears reading the same input share it). ``conv`` fuses the GatedDeltaNet causal
    conv of the leading ``conv_dim`` output rows into the epilogue. With ``comm`` the tensor-parallel sum is
    fused into the epilogue; ``push_only`` stops after publishing the partial rows (nothing is written to ``out``) and
    leaves the sum to ``add_rmsnorm_fp4_ar``: rows are left in this rank's multimem slot for an in-switch reduction
    when the communicator has a multicast address, else pushed to every rank as (value, epoch) pairs."""
    tw = prepare_fp4(q)
    assert n <= 16 and x16.shape[1] == tw.k
    bq, sfb, g0 = act if act is not None else quantize_act_fp4(x16, n, tw.kp)
    if out is None:
        out = torch.empty((n, tw.m), dtype=torch.float32 if out_f32 else torch.bfloat16, device=x16.device)
    rc = _lib.lib().vg_gemm_fp4(ptr(tw.wt), ptr(tw.row_scale), ptr(bq), c_int(bq.stride(0)), ptr(sfb), ptr(g0), ptr(out),
                                c_int(1 if out.dtype == torch.float32 else 0), c_int(tw.m), c_int(tw.k), c_int(n),
                                c_int(out.stride(0)), c_int(tw.splitk), ptr(_lib.err_word(x16.device)),
                                ctypes.byref(comm.ctx) if comm is not None else c_void_p(0),
                                c_int((2 if comm.use_mm else 1) if (push_only and comm is not None) else 0),
                                ctypes.byref(conv) if conv is not None else c_void_p(0), stream())
    _lib.check(rc, "vg_gemm_fp4")
    return out


def linear_fp4_grouped(q: QLinear, act, out: torch.Tensor, g_exp: torch.Tensor, g_off: torch.Tensor, n_items: int,
                       x_div: int, m_per_expert: int) -> torch.Tensor:
    """MoE decode on the FP4 path: work item g multiplies expert ``g_exp[g]`` (rows ``m_per_expert`` of the
    stacked tensor ``q``) with activation row ``g_off[g] // x_div`` of the quantised series ``act`` and writes
    ``out[g_off[g]]``. Items with ``g_exp < 0`` are skipped."""
    tw = prepare_fp4(q, splitk=1)
    bq, sfb, g0 = act
    rc = _lib.lib().vg_gemm_fp4_grouped(ptr(tw.wt), ptr(tw.row_scale), ptr(bq), c_int(bq.stride(0)), c_int(bq.shape[0]),
                                        ptr(sfb), ptr(g0), ptr(out), c_int(1 if out.dtype == torch.float32 else 0),
                                        c_int(m_per_expert), c_int(tw.k), c_int(out.stride(0)), c_int(n_items), ptr(g_exp),
                                        ptr(g_off), c_int(x_div), ptr(_lib.err_word(out.device)), stream())
    _lib.check(rc, "vg_gemm_fp4_grouped")
    return out

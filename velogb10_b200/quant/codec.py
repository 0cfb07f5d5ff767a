"""NVFP4 / FP8 weight-only codec (torch, vectorised; runs on CPU or CUDA tensors).

Bit-level contract, identical to the reference codec (reference: src/quant.rs:37-275):

* E2M1 magnitudes ``{0, .5, 1, 1.5, 2, 3, 4, 6}``, sign in bit 3, round-to-nearest with exact
  ties going to the even *code*.
* E4M3 is decoded as a float (bias 7, subnormals, no inf); the encoder picks the nearer of the two
  neighbouring codes and an exact tie goes to the lower code.
* NVFP4: block of 16 along K, ``global_scale = (6*448)/amax(W)`` stored in the *reciprocal*
  convention (dequant divides by it), block scale ``e4m3(amax(block)/6/s_tensor)``, packed two
  codes per byte with the low nibble holding the even index.
* FP8: one f32 scale per output row (``amax/448``), codes are E4M3.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

import torch

BLOCK = 16
E2M1_MAX = 6.0
E4M3_MAX = 448.0
E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def _e4m3_value(code: int) -> float:
    sign = -1.0 if code & 0x80 else 1.0
    exp = (code >> 3) & 0xF
    man = code & 0x7
    if exp == 0:
        return sign * (man / 8.0) * 2.0 ** -6
    return sign * (1.0 + man / 8.0) * 2.0 ** (exp - 7)


_E4M3_POS = torch.tensor([_e4m3_value(c) for c in range(127)], dtype=torch.float32)
_E4M3_ALL = torch.tensor([_e4m3_value(c) if (c & 0x7F) != 0x7F else float("nan")
                          for c in range(256)], dtype=torch.float32)
_E2M1_ALL = torch.tensor([(-v if c & 8 else v) for c in range(16) for v in [E2M1_VALUES[c & 7]]],
                         dtype=torch.float32)

_tables = {}


def _tab(t: torch.Tensor, device) -> torch.Tensor:
    key = (id(t), str(device))
    if key not in _tables:
        _tables[key] = t.to(device)
    return _tables[key]


# ------------------------------------------------------------------ scalar formats

def e4m3_decode(codes: torch.Tensor) -> torch.Tensor:
    """uint8 codes -> float32 values."""
    return _tab(_E4M3_ALL, codes.device)[codes.long()]


def e4m3_encode(x: torch.Tensor) -> torch.Tensor:
    """float32 -> uint8 E4M3 codes (nearest; tie -> lower code; non-finite / zero -> 0)."""
    x = x.float()
    t = _tab(_E4M3_POS, x.device)
    a = x.abs().clamp(max=E4M3_MAX)
    finite = torch.isfinite(x) & (x != 0)
    a = torch.where(finite, a, torch.zeros_like(a))
    hi = torch.searchsorted(t, a.contiguous(), right=False)
    hi_c = hi.clamp(1, 126)
    up = t[hi_c]
    lo = t[hi_c - 1]
    pick_hi = (up - a) < (a - lo)
    code = torch.where(pick_hi, hi_c, hi_c - 1)
    code = torch.where(hi == 0, torch.zeros_like(code), code)
    code = torch.where(hi >= 127, torch.full_like(code, 126), code)
    sign = (x < 0).to(torch.int64) << 7
    out = torch.where(finite, code | sign, torch.zeros_like(code))
    return out.to(torch.uint8)


def e2m1_decode(codes: torch.Tensor) -> torch.Tensor:
    return _tab(_E2M1_ALL, codes.device)[codes.long()]


def e2m1_encode(x: torch.Tensor) -> torch.Tensor:
    """float32 (already divided by the block scale) -> 4-bit codes in a uint8 tensor."""
    x = x.float()
    a = x.abs().clamp(max=E2M1_MAX)
    code = ((a > 0.25).to(torch.uint8) + (a >= 0.75).to(torch.uint8) + (a > 1.25).to(torch.uint8)
            + (a >= 1.75).to(torch.uint8) + (a > 2.5).to(torch.uint8) + (a >= 3.5).to(torch.uint8)
            + (a > 5.0).to(torch.uint8))
    return code | ((x < 0).to(torch.uint8) << 3)


# ------------------------------------------------------------------ NVFP4

@dataclass
class Nvfp4Tensor:
    """``weight_packed`` [M, K/2] u8, ``weight_scale`` [M, K/16] u8 (E4M3 codes),
    ``global_scale`` f32 scalar in the reciprocal convention."""
    packed: torch.Tensor
    scales: torch.Tensor
    global_scale: float
    m: int
    k: int


def quantize_nvfp4(w: torch.Tensor, amax: float | None = None, row_chunk: int = 8192) -> Nvfp4Tensor:
    """Quantize a [M, K] weight (bf16 or f32). ``amax`` may be given for a tensor that is
    processed in several pieces sharing one global scale (stacked experts)."""
    assert w.dim() == 2
    m, k = w.shape
    assert k % BLOCK == 0, f"K={k} is not a multiple of {BLOCK}"
    if amax is None:
        amax = float(w.abs().max().float()) if w.numel() else 0.0
    gs = torch.tensor((E2M1_MAX * E4M3_MAX) / amax if amax > 0 else 1.0, dtype=torch.float32)
    s_tensor = (torch.tensor(1.0, dtype=torch.float32) / gs).to(w.device)
    packed = torch.empty((m, k // 2), dtype=torch.uint8, device=w.device)
    scales = torch.empty((m, k // BLOCK), dtype=torch.uint8, device=w.device)
    for r0 in range(0, m, row_chunk):
        blk = w[r0:r0 + row_chunk].float().reshape(-1, k // BLOCK, BLOCK)
        bmax = blk.abs().amax(dim=-1)
        s_raw = torch.where(bmax > 0, bmax / E2M1_MAX / s_tensor, torch.zeros_like(bmax))
        s_code = e4m3_encode(s_raw)
        s = e4m3_decode(s_code) * s_tensor
        inv = torch.where(s > 0, 1.0 / s, torch.zeros_like(s))
        q = e2m1_encode(blk * inv.unsqueeze(-1)).reshape(-1, k)
        packed[r0:r0 + row_chunk] = q[:, 0::2] | (q[:, 1::2] << 4)
        scales[r0:r0 + row_chunk] = s_code
    return Nvfp4Tensor(packed, scales, float(gs), m, k)


def dequantize_nvfp4(packed: torch.Tensor, scales: torch.Tensor, global_scale: float,
                     dtype=torch.bfloat16) -> torch.Tensor:
    m, kh = packed.shape
    k = kh * 2
    s_tensor = (torch.tensor(1.0, dtype=torch.float32) / torch.tensor(global_scale, dtype=torch.float32))
    s = e4m3_decode(scales) * s_tensor.to(packed.device)
    codes = torch.stack([packed & 0xF, packed >> 4], dim=-1).reshape(m, k)
    vals = e2m1_decode(codes).reshape(m, k // BLOCK, BLOCK) * s.unsqueeze(-1)
    return vals.reshape(m, k).to(dtype)


# ------------------------------------------------------------------ FP8 per-row

@dataclass
class Fp8Tensor:
    codes: torch.Tensor      # [M, K] u8
    row_scale: torch.Tensor  # [M] f32
    m: int
    k: int


def quantize_fp8(w: torch.Tensor, row_chunk: int = 8192) -> Fp8Tensor:
    m, k = w.shape
    codes = torch.empty((m, k), dtype=torch.uint8, device=w.device)
    row_scale = torch.empty((m,), dtype=torch.float32, device=w.device)
    for r0 in range(0, m, row_chunk):
        x = w[r0:r0 + row_chunk].float()
        amax = x.abs().amax(dim=-1)
        s = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
        row_scale[r0:r0 + row_chunk] = s
        codes[r0:r0 + row_chunk] = e4m3_encode(x * (1.0 / s).unsqueeze(-1))
    return Fp8Tensor(codes, row_scale, m, k)


def dequantize_fp8(codes: torch.Tensor, row_scale: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    return (e4m3_decode(codes) * row_scale.float().unsqueeze(-1)).to(dtype)


# ------------------------------------------------------------------ helpers

def fake_quant(w: torch.Tensor, fmt: str) -> torch.Tensor:
    """Round-trip ``w`` through a format; the result keeps ``w``'s dtype."""
    if fmt == "bf16":
        return w
    w2 = w.reshape(-1, w.shape[-1])
    if fmt == "nvfp4":
        q = quantize_nvfp4(w2)
        out = dequantize_nvfp4(q.packed, q.scales, q.global_scale, w.dtype)
    elif fmt == "fp8":
        q8 = quantize_fp8(w2)
        out = dequantize_fp8(q8.codes, q8.row_scale, w.dtype)
    else:
        raise ValueError(fmt)
    return out.reshape(w.shape)


def bits_per_weight(fmt: str, k: int) -> float:
    return {"bf16": 16.0, "fp8": 8.0 + 32.0 / k, "nvfp4": 4.0 + 8.0 / BLOCK}[fmt]


def roundtrip_error(orig: torch.Tensor, deq: torch.Tensor) -> Tuple[float, float]:
    a, b = orig.double(), deq.double()
    rel = float(((a - b).pow(2).sum() / a.pow(2).sum().clamp(min=1e-30)).sqrt())
    return rel, float((a - b).abs().max())

// Device helpers of the four-term NVFP4 activation quantiser, shared by the stand-alone quantiser kernels and
// by producers that quantise their own output (layout described in act_quant.cu).
#pragma once
#include "common.cuh"

namespace vg {
namespace aq {

constexpr int TERMS = 4;
constexpr int SF_BYTES = 2048;

__device__ __forceinline__ uint8_t f32_to_e4m3(float v) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.0f), "f"(v));
  return (uint8_t)(r & 0xff);
}
__device__ __forceinline__ float e4m3_to_f32(uint8_t c) {
  uint32_t h;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h) : "h"((uint16_t)c));
  return __half22float2(*reinterpret_cast<__half2*>(&h)).x;
}
__device__ __forceinline__ uint32_t f32x2_to_e2m1x2(float lo, float hi) {
  uint32_t r;
  asm("{\n\t.reg .b8 b0;\n\tcvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\tcvt.u32.u8 %0, b0;\n\t}\n" : "=r"(r) : "f"(lo), "f"(hi));
  return r & 0xffu;
}
__device__ __forceinline__ float2 e2m1x2_to_f32(uint32_t c) {
  uint32_t h;
  asm("{\n\t.reg .b8 b0;\n\tcvt.u8.u32 b0, %1;\n\tcvt.rn.f16x2.e2m1x2 %0, b0;\n\t}\n" : "=r"(h) : "r"(c));
  return __half22float2(*reinterpret_cast<__half2*>(&h));
}
// eight values -> four bytes of e2m1 codes (low nibble = first element of each pair)
__device__ __forceinline__ uint32_t f32x8_to_e2m1(const float* v) {
  return f32x2_to_e2m1x2(v[0], v[1]) | (f32x2_to_e2m1x2(v[2], v[3]) << 8) | (f32x2_to_e2m1x2(v[4], v[5]) << 16) |
         (f32x2_to_e2m1x2(v[6], v[7]) << 24);
}
__device__ __forceinline__ void e2m1x8_to_f32(uint32_t w, float* o) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = e2m1x2_to_f32((w >> (8 * i)) & 0xffu);
    o[2 * i] = f.x;
    o[2 * i + 1] = f.y;
  }
}

__device__ __forceinline__ float rcp_approx(float x) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

// Quantise one 16-element block (values in r, consumed) of row n, block index b, into the four terms.
// Rows are grouped sixteen to a 64-row B tile: row n lives in tile n / 16 as column n % 16 (tile T starts at
// bq row 64 T and at scale chunk T * (ldb / 128)).
// This routine sits on the serial path of every decode-width producer (a thread runs its four terms back to back),
// so it is written for a short dependent chain: the block maximum as a tree, one true division per call (the
// per-term scale factors are exact multiples of 8 of it), the hardware reciprocal for the element scaling (the
// residual is formed from the codes actually stored, so the series stays exact whatever the rounding of a term).
__device__ __forceinline__ void quant_block(float* r, float g, int n, int b, uint8_t* __restrict__ bq, int ldb,
                                            uint8_t* __restrict__ sfb) {
  const int slab = b >> 4, step = (b & 15) >> 2, kb = b & 3;
  const int tile = n >> 4;
  n &= 15;
  bq += (size_t)tile * 64 * ldb;
  sfb += (size_t)tile * (ldb >> 7) * SF_BYTES;
  float gt = g;
  float q6 = 1.0f / (6.0f * g);            // block maximum -> scale code, term 0; times 8 per further term
#pragma unroll
  for (int t = 0; t < TERMS; ++t) {
    float m[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) m[i] = fmaxf(fabsf(r[2 * i]), fabsf(r[2 * i + 1]));
    const float bmax = fmaxf(fmaxf(fmaxf(m[0], m[1]), fmaxf(m[2], m[3])), fmaxf(fmaxf(m[4], m[5]), fmaxf(m[6], m[7])));
    const uint8_t sc = f32_to_e4m3(bmax * q6);
    const float s = e4m3_to_f32(sc) * gt;
    const float inv = s > 0.f ? rcp_approx(s) : 0.f;
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = r[i] * inv;
    const uint32_t w0 = f32x8_to_e2m1(v), w1 = f32x8_to_e2m1(v + 8);
    float d[16];
    e2m1x8_to_f32(w0, d);
    e2m1x8_to_f32(w1, d + 8);
#pragma unroll
    for (int i = 0; i < 16; ++i) r[i] = fmaf(-d[i], s, r[i]);
    const int row = t * 16 + n;
    *reinterpret_cast<uint2*>(bq + (size_t)row * ldb + b * 8) = make_uint2(w0, w1);
    sfb[(size_t)slab * SF_BYTES + step * 512 + (row & 31) * 16 + (row >> 5) * 4 + kb] = sc;
    gt *= 0.125f;
    q6 *= 8.0f;
  }
}

__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = (threadIdx.x & 31) < ((blockDim.x + 31) >> 5) ? red[threadIdx.x & 31] : 0.f;
  return warp_max(t);
}

}  // namespace aq
}  // namespace vg

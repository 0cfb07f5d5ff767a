// Activation quantiser for the block-scaled FP4 GEMM: each f16 row (token column) becomes a four-term NVFP4
// residual series. One CTA per row; a thread owns whole 16-element blocks, keeps them in registers from the
// single global read through the row-maximum reduction to the four quantisation rounds, so the only
// cross-thread step is one block-wide max. Fused variants do the same at the end of RMSNorm and SwiGLU, whose
// outputs are GEMM inputs, so those rows never round-trip through memory in f16.
//
// Output layout (shared with gemm_fp4.cu):
//   bq   [64][ldb bytes]  row t*16 + n = term t of row n, two e2m1 codes per byte (low nibble = even k)
//   sfb  [K/256][4][512]  scale chunks: byte [r0*16 + r1*4 + kb] of step j = e4m3 scale of bq row
//                         (r0 + 32*r1), 16-element block j*4 + kb of the slab
//   g0   [16]             amax / (6 * 448) of each row; term t uses the global scale g0 / 8^t
// Rows >= N are left untouched: their accumulator columns are never stored.
#include "common.cuh"
#include "api.h"

namespace {
using namespace vg;

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

// Quantise one 16-element block (values in r, consumed) of row n, block index b, into the four terms.
__device__ __forceinline__ void quant_block(float* r, float g, int n, int b, uint8_t* __restrict__ bq, int ldb,
                                            uint8_t* __restrict__ sfb) {
  const int slab = b >> 4, step = (b & 15) >> 2, kb = b & 3;
  float gt = g;
#pragma unroll
  for (int t = 0; t < TERMS; ++t) {
    float bmax = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) bmax = fmaxf(bmax, fabsf(r[i]));
    const uint8_t sc = f32_to_e4m3(bmax / (6.0f * gt));
    const float s = e4m3_to_f32(sc) * gt;
    const float inv = s > 0.f ? 1.0f / s : 0.f;
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

constexpr int MAXB = 3;     // 16-element blocks a thread may hold

// mode 0: x is the f16 row.  mode 1: SwiGLU of a bf16 [gate | up] row.  Both: quantise to FP4 terms.
template <int MODE>
__global__ void __launch_bounds__(1024) act_quant_kernel(const void* __restrict__ xin, int ldx, int K, int Kpad,
                                                          uint8_t* __restrict__ bq, int ldb, uint8_t* __restrict__ sfb,
                                                          float* __restrict__ g0, __half* __restrict__ out16) {
  __shared__ float red[32];
  const int n = blockIdx.x;
  const int nblk = Kpad >> 4;
  float r[MAXB][16];
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < MAXB; ++j) {
    const int b = threadIdx.x + j * blockDim.x;
    if (b < nblk) {
      const int k0 = b * 16;
      if (k0 + 16 <= K) {
        if (MODE == 0) {
          const uint4* src = reinterpret_cast<const uint4*>(static_cast<const __half*>(xin) + (size_t)n * ldx + k0);
          const uint4 a = src[0], c = src[1];
          const __half2* ha = reinterpret_cast<const __half2*>(&a);
          const __half2* hc = reinterpret_cast<const __half2*>(&c);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 fa = __half22float2(ha[i]), fc = __half22float2(hc[i]);
            r[j][2 * i] = fa.x; r[j][2 * i + 1] = fa.y; r[j][8 + 2 * i] = fc.x; r[j][8 + 2 * i + 1] = fc.y;
          }
        } else {
          const __nv_bfloat16* gp = static_cast<const __nv_bfloat16*>(xin) + (size_t)n * ldx + k0;
          const __nv_bfloat16* up = gp + K;
          const uint4 g0v = reinterpret_cast<const uint4*>(gp)[0], g1v = reinterpret_cast<const uint4*>(gp)[1];
          const uint4 u0v = reinterpret_cast<const uint4*>(up)[0], u1v = reinterpret_cast<const uint4*>(up)[1];
          const __nv_bfloat16* gg0 = reinterpret_cast<const __nv_bfloat16*>(&g0v);
          const __nv_bfloat16* gg1 = reinterpret_cast<const __nv_bfloat16*>(&g1v);
          const __nv_bfloat16* uu0 = reinterpret_cast<const __nv_bfloat16*>(&u0v);
          const __nv_bfloat16* uu1 = reinterpret_cast<const __nv_bfloat16*>(&u1v);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            r[j][i] = __half2float(f32_to_f16_sat(silu(__bfloat162float(gg0[i])) * __bfloat162float(uu0[i])));
            r[j][8 + i] = __half2float(f32_to_f16_sat(silu(__bfloat162float(gg1[i])) * __bfloat162float(uu1[i])));
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int k = k0 + i;
          float v = 0.f;
          if (k < K) {
            if (MODE == 0) v = __half2float(static_cast<const __half*>(xin)[(size_t)n * ldx + k]);
            else {
              const __nv_bfloat16* gp = static_cast<const __nv_bfloat16*>(xin) + (size_t)n * ldx;
              v = __half2float(f32_to_f16_sat(silu(__bfloat162float(gp[k])) * __bfloat162float(gp[K + k])));
            }
          }
          r[j][i] = v;
        }
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(r[j][i]));
      if (out16 && k0 + 16 <= K) {
        uint4 o0, o1;
        __half* h0 = reinterpret_cast<__half*>(&o0);
        __half* h1 = reinterpret_cast<__half*>(&o1);
#pragma unroll
        for (int i = 0; i < 8; ++i) { h0[i] = __float2half_rn(r[j][i]); h1[i] = __float2half_rn(r[j][8 + i]); }
        uint4* dst = reinterpret_cast<uint4*>(out16 + (size_t)n * K + k0);
        dst[0] = o0; dst[1] = o1;
      }
    }
  }
  amax = block_max(amax, red);
  const float g = amax > 0.f ? amax / (6.0f * 448.0f) : 1.0f;
  if (threadIdx.x == 0) g0[n] = g;
#pragma unroll
  for (int j = 0; j < MAXB; ++j) {
    const int b = threadIdx.x + j * blockDim.x;
    if (b < nblk) quant_block(r[j], g, n, b, bq, ldb, sfb);
  }
}

// residual += delta; y = rmsnorm(residual) * (1 + w); emit y as FP4 terms (and optionally as f16).
__global__ void __launch_bounds__(1024) add_rmsnorm_fp4_kernel(__nv_bfloat16* res, const __nv_bfloat16* delta, const float* w,
                                                                int h, float eps, int plus_one, int ld_res, int ld_delta,
                                                                int Kpad, uint8_t* __restrict__ bq, int ldb,
                                                                uint8_t* __restrict__ sfb, float* __restrict__ g0,
                                                                __half* __restrict__ out16) {
  __shared__ float red[32];
  const int n = blockIdx.x;
  __nv_bfloat16* rp = res + (size_t)n * ld_res;
  const __nv_bfloat16* dp = delta ? delta + (size_t)n * ld_delta : nullptr;
  const int nblk = Kpad >> 4, hblk = h >> 4;
  float r[MAXB][16];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < MAXB; ++j) {
    const int b = threadIdx.x + j * blockDim.x;
#pragma unroll
    for (int i = 0; i < 16; ++i) r[j][i] = 0.f;
    if (b < hblk) {
      const uint4 a0 = reinterpret_cast<const uint4*>(rp + b * 16)[0], a1 = reinterpret_cast<const uint4*>(rp + b * 16)[1];
      uint4 d0 = make_uint4(0, 0, 0, 0), d1 = d0;
      if (dp) { d0 = reinterpret_cast<const uint4*>(dp + b * 16)[0]; d1 = reinterpret_cast<const uint4*>(dp + b * 16)[1]; }
      const __nv_bfloat16* x0 = reinterpret_cast<const __nv_bfloat16*>(&a0);
      const __nv_bfloat16* x1 = reinterpret_cast<const __nv_bfloat16*>(&a1);
      const __nv_bfloat16* y0 = reinterpret_cast<const __nv_bfloat16*>(&d0);
      const __nv_bfloat16* y1 = reinterpret_cast<const __nv_bfloat16*>(&d1);
      uint4 u0, u1;
      __nv_bfloat16* o0 = reinterpret_cast<__nv_bfloat16*>(&u0);
      __nv_bfloat16* o1 = reinterpret_cast<__nv_bfloat16*>(&u1);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float v0 = __bfloat162float(x0[i]), v1 = __bfloat162float(x1[i]);
        if (dp) {
          o0[i] = __float2bfloat16_rn(v0 + __bfloat162float(y0[i]));
          o1[i] = __float2bfloat16_rn(v1 + __bfloat162float(y1[i]));
          v0 = __bfloat162float(o0[i]); v1 = __bfloat162float(o1[i]);
        }
        r[j][i] = v0; r[j][8 + i] = v1;
        ss += v0 * v0 + v1 * v1;
      }
      if (dp) { reinterpret_cast<uint4*>(rp + b * 16)[0] = u0; reinterpret_cast<uint4*>(rp + b * 16)[1] = u1; }
    }
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)h + eps);
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < MAXB; ++j) {
    const int b = threadIdx.x + j * blockDim.x;
    if (b < hblk) {
      uint4 o0, o1;
      __half* h0 = reinterpret_cast<__half*>(&o0);
      __half* h1 = reinterpret_cast<__half*>(&o1);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float wv = w[b * 16 + i];
        // round through f16 so both outputs describe the same values
        const __half y = f32_to_f16_sat(r[j][i] * inv * (plus_one ? 1.0f + wv : wv));
        if (i < 8) h0[i] = y; else h1[i - 8] = y;
        r[j][i] = __half2float(y);
        amax = fmaxf(amax, fabsf(r[j][i]));
      }
      if (out16) { reinterpret_cast<uint4*>(out16 + (size_t)n * h + b * 16)[0] = o0; reinterpret_cast<uint4*>(out16 + (size_t)n * h + b * 16)[1] = o1; }
    }
  }
  amax = block_max(amax, red);
  const float g = amax > 0.f ? amax / (6.0f * 448.0f) : 1.0f;
  if (threadIdx.x == 0) g0[n] = g;
#pragma unroll
  for (int j = 0; j < MAXB; ++j) {
    const int b = threadIdx.x + j * blockDim.x;
    if (b < nblk) quant_block(r[j], g, n, b, bq, ldb, sfb);
  }
}

int threads_for(int nblk) {
  int t = (nblk + 31) / 32 * 32;
  if (t > 1024) t = (((nblk + MAXB - 1) / MAXB) + 31) / 32 * 32;
  return t < 32 ? 32 : t;
}

}  // namespace

// x [N <= 16, K] f16 (row stride ldx) -> FP4 terms. Kpad = ldb * 2 must be a multiple of 256 and >= K.
extern "C" int vg_act_quant_fp4(const void* x_f16, int ldx, int N, int K, void* bq, int ldb, void* sfb, float* g0,
                                cudaStream_t st) {
  const int Kpad = ldb * 2;
  if (N < 1 || N > 16 || (ldb % 128) != 0 || Kpad < K || (K % 8) != 0 || (ldx % 8) != 0 || (Kpad >> 4) > 1024 * MAXB) return -2;
  act_quant_kernel<0><<<N, threads_for(Kpad >> 4), 0, st>>>(x_f16, ldx, K, Kpad, static_cast<uint8_t*>(bq), ldb,
                                                            static_cast<uint8_t*>(sfb), g0, nullptr);
  return (int)cudaGetLastError();
}

// gu [N, 2*I] bf16 (row stride ld) -> SwiGLU -> FP4 terms (and f16 copy when out16 != null, [N, I] contiguous).
extern "C" int vg_swiglu_fp4(const void* gu, int ld, int N, int I, void* bq, int ldb, void* sfb, float* g0, void* out16,
                             cudaStream_t st) {
  const int Kpad = ldb * 2;
  if (N < 1 || N > 16 || (ldb % 128) != 0 || Kpad < I || (I % 8) != 0 || (ld % 8) != 0 || (Kpad >> 4) > 1024 * MAXB) return -2;
  act_quant_kernel<1><<<N, threads_for(Kpad >> 4), 0, st>>>(gu, ld, I, Kpad, static_cast<uint8_t*>(bq), ldb,
                                                            static_cast<uint8_t*>(sfb), g0, static_cast<__half*>(out16));
  return (int)cudaGetLastError();
}

extern "C" int vg_add_rmsnorm_fp4(void* res, const void* delta, const float* w, int N, int h, float eps, int plus_one,
                                  int ld_res, int ld_delta, void* bq, int ldb, void* sfb, float* g0, void* out16,
                                  cudaStream_t st) {
  const int Kpad = ldb * 2;
  if (N < 1 || N > 16 || (ldb % 128) != 0 || Kpad < h || (h % 16) != 0 || (ld_res % 8) != 0 || (ld_delta % 8) != 0 ||
      (Kpad >> 4) > 1024 * MAXB)
    return -2;
  add_rmsnorm_fp4_kernel<<<N, threads_for(Kpad >> 4), 0, st>>>(static_cast<__nv_bfloat16*>(res),
                                                               static_cast<const __nv_bfloat16*>(delta), w, h, eps, plus_one,
                                                               ld_res, ld_delta, Kpad, static_cast<uint8_t*>(bq), ldb,
                                                               static_cast<uint8_t*>(sfb), g0, static_cast<__half*>(out16));
  return (int)cudaGetLastError();
}

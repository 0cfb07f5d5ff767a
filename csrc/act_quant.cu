// Activation quantiser for the block-scaled FP4 GEMM: each f16 row (token column) becomes a four-term NVFP4
// residual series. One CTA per row; a thread owns whole 16-element blocks, keeps them in registers from the
// single global read through the row-maximum reduction to the four quantisation rounds, so the only
// cross-thread step is one block-wide max. Fused variants do the same at the end of RMSNorm and SwiGLU, whose
// outputs are GEMM inputs, so those rows never round-trip through memory in f16.
//
// Output layout (shared with gemm_fp4.cu):
//   bq   [64][ldb bytes]  row t*16 + n = term t of row n, two e2m1 codes per byte (low nibble = even k);
//                         rows 16.. of the stand-alone quantisers continue in further 64-row tiles (grouped GEMM)
//   sfb  [K/256][4][512]  scale chunks: byte [r0*16 + r1*4 + kb] of step j = e4m3 scale of bq row
//                         (r0 + 32*r1), 16-element block j*4 + kb of the slab
//   g0   [16]             amax / (6 * 448) of each row; term t uses the global scale g0 / 8^t
// Rows >= N are left untouched: their accumulator columns are never stored.
#include "common.cuh"
#include "act_quant.cuh"
#include "api.h"

namespace {
using namespace vg;

using namespace vg::aq;

constexpr int MAXB = 3;     // 16-element blocks a thread may hold

// mode 0: x is the f16 row.  mode 1: SwiGLU of a bf16 [gate | up] row.  Both: quantise to FP4 terms.
template <int MODE>
__global__ void __launch_bounds__(512) act_quant_kernel(const void* __restrict__ xin, int ldx, int K, int Kpad,
                                                          uint8_t* __restrict__ bq, int ldb, uint8_t* __restrict__ sfb,
                                                          float* __restrict__ g0, __half* __restrict__ out16) {
  __shared__ float red[32];
  if (threadIdx.x == 0) trace(32);
  if (gridDim.x > 1) cluster_arrive_relaxed();
  pdl_trigger();
  pdl_wait();
  if (threadIdx.x == 0) trace(33);
  // a cluster of gridDim.x CTAs shares one row: CTA c owns blocks [c * bpc, (c + 1) * bpc)
  __shared__ float cl_amax[8];
  const int n = blockIdx.y, C = gridDim.x, c = blockIdx.x;
  const int nblk = Kpad >> 4;
  const int bpc = (nblk + C - 1) / C;
  const int b_end = min(nblk, (c + 1) * bpc);
  float r[MAXB][16];
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < MAXB; ++j) {
    const int b = c * bpc + threadIdx.x + j * blockDim.x;
    if (b < b_end) {
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
  if (threadIdx.x == 0) trace(2 * 16 + 3);
  if (C > 1) {
    // every CTA stores its maximum into slot c of every CTA of the cluster (its own included); one cluster barrier
    // orders the stores before the reads, which are local, so nobody touches a peer's memory after the barrier
    cluster_wait();                                        // pairs with the arrive at entry: every peer has started
    if (threadIdx.x < C) dsmem_st_f32(dsmem_map(smem_u32(&cl_amax[c]), threadIdx.x), amax);
    cluster_sync_all();
    for (int q = 0; q < C; ++q) amax = fmaxf(amax, cl_amax[q]);
  }
  if (threadIdx.x == 0) trace(2 * 16 + 4);
  const float g = amax > 0.f ? amax / (6.0f * 448.0f) : 1.0f;
  if (threadIdx.x == 0 && c == 0) g0[n] = g;
#pragma unroll
  for (int j = 0; j < MAXB; ++j) {
    const int b = c * bpc + threadIdx.x + j * blockDim.x;
    if (b < b_end) quant_block(r[j], g, n, b, bq, ldb, sfb);
  }
  if (threadIdx.x == 0) trace(2 * 16 + 2);
}

// residual += delta; y = rmsnorm(residual) * (1 + w); emit y as FP4 terms (and optionally as f16).
// AR: delta is not a tensor but the sum over ranks of the fp32 partial rows in this rank's receive slots
// (pushed there by every rank's row-parallel GEMM); the kernel waits for the tile flags and sums in rank order.
// AR = 2: delta is the in-switch sum (multimem.ld_reduce) of the rows every rank's GEMM left in its own multimem slot.
template <int AR>
__global__ void __launch_bounds__(512) add_rmsnorm_fp4_kernel(__nv_bfloat16* res, const __nv_bfloat16* delta, const float* w,
                                                                int h, float eps, int plus_one, int ld_res, int ld_delta,
                                                                int Kpad, uint8_t* __restrict__ bq, int ldb,
                                                                uint8_t* __restrict__ sfb, float* __restrict__ g0,
                                                                __half* __restrict__ out16, const VgCommCtx c) {
  __shared__ float red[32];
  if (threadIdx.x == 0) trace(16);
  pdl_trigger();
  // the norm weights do not depend on the preceding kernel: fetch the first block's before waiting for it
  float4 w0[4];
  {
    const int hb = h >> 4;
    const float4* wp = reinterpret_cast<const float4*>(w + (size_t)min((int)threadIdx.x, hb - 1) * 16);
#pragma unroll
    for (int i = 0; i < 4; ++i) w0[i] = wp[i];
  }
  pdl_wait();
  if (threadIdx.x == 0) trace(17);
  const int n = blockIdx.x;
  __nv_bfloat16* rp = res + (size_t)n * ld_res;
  const __nv_bfloat16* dp = (!AR && delta) ? delta + (size_t)n * ld_delta : nullptr;
  const int nblk = Kpad >> 4, hblk = h >> 4;
  uint32_t ar_e = 0;
  int ar_set = 0;
  if (AR) {
    ar_e = *c.epoch + 1;
    ar_set = ar_e & 1;
  }
  const uint32_t* mm_flags = AR == 2 ? reinterpret_cast<const uint32_t*>(c.data[c.rank] + c.mmflags_off) + (size_t)ar_set * MAX_CTAS * MAX_RANKS
                                       : nullptr;
  float r[MAXB][16];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < MAXB; ++j) {
    const int b = threadIdx.x + j * blockDim.x;
#pragma unroll
    for (int i = 0; i < 16; ++i) r[j][i] = 0.f;
    if (b < hblk) {
      const uint4 a0 = reinterpret_cast<const uint4*>(rp + b * 16)[0], a1 = reinterpret_cast<const uint4*>(rp + b * 16)[1];
      const __nv_bfloat16* x0 = reinterpret_cast<const __nv_bfloat16*>(&a0);
      const __nv_bfloat16* x1 = reinterpret_cast<const __nv_bfloat16*>(&a1);
      float dv[16];
      bool have_d = dp != nullptr;
      if (AR == 2) {
        // the 128-row GEMM tile these 16 elements belong to: wait (bounded) until every rank's word for the tile
        // carries this collective's epoch, then read the in-switch sum of the W copies
        // (the tile's MAX_RANKS words are one 32-byte line: two volatile 16-byte loads fetch them all in one L2 round
        // trip, where an acquire load per word would wait for the one before. The data reads that follow depend on
        // the branch on these words and go to the switch, not to a local cache, and every writer fences at system
        // scope before its word: the flag-then-data order holds without a reader-side fence, which measured 3 us.)
        const uint4* f = reinterpret_cast<const uint4*>(mm_flags + (size_t)(b >> 3) * MAX_RANKS);
        bool ok = false;
        uint64_t t_start = 0;
        for (int tries = 0;; ++tries) {
          uint4 fa, fb;
          asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(fa.x), "=r"(fa.y), "=r"(fa.z), "=r"(fa.w) : "l"(f) : "memory");
          asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(fb.x), "=r"(fb.y), "=r"(fb.z), "=r"(fb.w) : "l"(f + 1) : "memory");
          const uint32_t fw[MAX_RANKS] = {fa.x, fa.y, fa.z, fa.w, fb.x, fb.y, fb.z, fb.w};
          ok = true;
#pragma unroll
          for (int q = 0; q < MAX_RANKS; ++q) ok = ok && (q >= c.world || (int32_t)(fw[q] - ar_e) >= 0);
          if (ok) break;
          if (tries == 64) t_start = global_ns();
          if (tries > 64 && (tries & 63) == 0 && global_ns() - t_start > c.timeout_ns) {
            atomicCAS(c.status, 0, VG_ERR_PEER_WAIT);
            break;
          }
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) dv[i] = 0.f;
        if (ok) {
          const unsigned char* src = c.mc + c.mm_off + (size_t)ar_set * c.mm_slot_bytes + ((size_t)n * h + b * 16) * 4;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float4 v = multimem_ld_reduce_f32x4(src + 16 * i);
            dv[4 * i] = v.x; dv[4 * i + 1] = v.y; dv[4 * i + 2] = v.z; dv[4 * i + 3] = v.w;
          }
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) dv[i] = __bfloat162float(__float2bfloat16_rn(dv[i]));
        have_d = true;
      } else if (AR == 1) {
        // Every rank stored its (value, epoch) pairs for these 16 elements into this rank's receive slots: poll
        // them (local memory) and take them once all 16 carry this collective's epoch; sum in rank order.
        // Bounded by the context's timeout.
        const size_t stride = c.slot_bytes;
#pragma unroll
        for (int i = 0; i < 16; ++i) dv[i] = 0.f;
        // Two ranks' pairs are fetched per poll round (sixteen independent 16-byte loads in flight), so the wait
        // costs world / 2 round trips to L2 instead of world; the sums still run in rank order.
        for (int q = 0; q < c.world; q += 2) {
          const uint4* src0 = reinterpret_cast<const uint4*>(c.data[c.rank] + c.slots_off + (size_t)(ar_set * MAX_RANKS + q) * stride) +
                              (((size_t)n * h + b * 16) >> 1);
          const bool two = q + 1 < c.world;
          const uint4* src1 = two ? reinterpret_cast<const uint4*>(c.data[c.rank] + c.slots_off + (size_t)(ar_set * MAX_RANKS + q + 1) * stride) +
                                        (((size_t)n * h + b * 16) >> 1)
                                  : src0;
          uint4 v[8], w[8];
          uint64_t t_start = 0;
          for (int tries = 0;; ++tries) {
            bool ok = true;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                           : "=r"(v[i].x), "=r"(v[i].y), "=r"(v[i].z), "=r"(v[i].w) : "l"(src0 + i) : "memory");
              asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                           : "=r"(w[i].x), "=r"(w[i].y), "=r"(w[i].z), "=r"(w[i].w) : "l"(src1 + i) : "memory");
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) ok = ok && v[i].y == ar_e && v[i].w == ar_e && w[i].y == ar_e && w[i].w == ar_e;
            if (ok) break;
            if (tries == 64) t_start = global_ns();
            if (tries > 64 && (tries & 63) == 0 && global_ns() - t_start > c.timeout_ns) {
              atomicCAS(c.status, 0, VG_ERR_PEER_WAIT);
              break;
            }
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) { dv[2 * i] += __uint_as_float(v[i].x); dv[2 * i + 1] += __uint_as_float(v[i].z); }
          if (two) {
#pragma unroll
            for (int i = 0; i < 8; ++i) { dv[2 * i] += __uint_as_float(w[i].x); dv[2 * i + 1] += __uint_as_float(w[i].z); }
          }
        }
        // the unfused path stores the sum as bf16 before the residual add: keep the same rounding
#pragma unroll
        for (int i = 0; i < 16; ++i) dv[i] = __bfloat162float(__float2bfloat16_rn(dv[i]));
        have_d = true;
      } else if (dp) {
        const uint4 d0 = reinterpret_cast<const uint4*>(dp + b * 16)[0], d1 = reinterpret_cast<const uint4*>(dp + b * 16)[1];
        const __nv_bfloat16* y0 = reinterpret_cast<const __nv_bfloat16*>(&d0);
        const __nv_bfloat16* y1 = reinterpret_cast<const __nv_bfloat16*>(&d1);
#pragma unroll
        for (int i = 0; i < 8; ++i) { dv[i] = __bfloat162float(y0[i]); dv[8 + i] = __bfloat162float(y1[i]); }
      }
      uint4 u0, u1;
      __nv_bfloat16* o0 = reinterpret_cast<__nv_bfloat16*>(&u0);
      __nv_bfloat16* o1 = reinterpret_cast<__nv_bfloat16*>(&u1);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float v0 = __bfloat162float(x0[i]), v1 = __bfloat162float(x1[i]);
        if (have_d) {
          o0[i] = __float2bfloat16_rn(v0 + dv[i]);
          o1[i] = __float2bfloat16_rn(v1 + dv[8 + i]);
          v0 = __bfloat162float(o0[i]); v1 = __bfloat162float(o1[i]);
        }
        r[j][i] = v0; r[j][8 + i] = v1;
        ss += v0 * v0 + v1 * v1;
      }
      if (have_d) { reinterpret_cast<uint4*>(rp + b * 16)[0] = u0; reinterpret_cast<uint4*>(rp + b * 16)[1] = u1; }
    }
  }
  ss = block_sum(ss, red);
  if (threadIdx.x == 0) trace(1 * 16 + 3);
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
        const float wv = j == 0 ? reinterpret_cast<const float*>(w0)[i] : w[b * 16 + i];
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
  if (threadIdx.x == 0) trace(1 * 16 + 4);
  const float g = amax > 0.f ? amax / (6.0f * 448.0f) : 1.0f;
  if (threadIdx.x == 0) g0[n] = g;
#pragma unroll
  for (int j = 0; j < MAXB; ++j) {
    const int b = threadIdx.x + j * blockDim.x;
    if (b < nblk) quant_block(r[j], g, n, b, bq, ldb, sfb);
  }
  if (AR) {
    // every row has consumed the slots: the last CTA publishes the epoch for the next collective
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      if (atomicAdd(c.done_ctr, 1u) == gridDim.x - 1) { *c.done_ctr = 0; *c.epoch = ar_e; }
    }
  }
  if (threadIdx.x == 0) trace(1 * 16 + 2);
}

constexpr int MAX_THREADS = 512;
int threads_for(int nblk) {
  int t = (nblk + 31) / 32 * 32;
  if (t > MAX_THREADS) t = (((nblk + MAXB - 1) / MAXB) + 31) / 32 * 32;
  return t < 32 ? 32 : t;
}
// CTAs per row for the stand-alone quantisers: about 128 blocks per CTA, at most a portable cluster.
int cluster_for(int nblk) {
  int c = (nblk + 127) / 128;
  return c < 1 ? 1 : (c > 8 ? 8 : c);
}

}  // namespace

// x [N <= 16, K] f16 (row stride ldx) -> FP4 terms. Kpad = ldb * 2 must be a multiple of 256 and >= K.
extern "C" int vg_act_quant_fp4(const void* x_f16, int ldx, int N, int K, void* bq, int ldb, void* sfb, float* g0,
                                cudaStream_t st) {
  const int Kpad = ldb * 2;
  if (N < 1 || N > 4096 || (ldb % 128) != 0 || Kpad < K || (K % 8) != 0 || (ldx % 8) != 0 || (Kpad >> 4) > MAX_THREADS * MAXB) return -2;
  const int C = cluster_for(Kpad >> 4), bpc = ((Kpad >> 4) + C - 1) / C;
  return (int)launch_pdl_cluster(act_quant_kernel<0>, dim3(C, N), dim3(threads_for(bpc)), (unsigned)C, 0, st, x_f16, ldx, K,
                                 Kpad, static_cast<uint8_t*>(bq), ldb, static_cast<uint8_t*>(sfb), g0, (__half*)nullptr);
}

// gu [N, 2*I] bf16 (row stride ld) -> SwiGLU -> FP4 terms (and f16 copy when out16 != null, [N, I] contiguous).
extern "C" int vg_swiglu_fp4(const void* gu, int ld, int N, int I, void* bq, int ldb, void* sfb, float* g0, void* out16,
                             cudaStream_t st) {
  const int Kpad = ldb * 2;
  if (N < 1 || N > 4096 || (ldb % 128) != 0 || Kpad < I || (I % 8) != 0 || (ld % 8) != 0 || (Kpad >> 4) > MAX_THREADS * MAXB) return -2;
  const int C = cluster_for(Kpad >> 4), bpc = ((Kpad >> 4) + C - 1) / C;
  return (int)launch_pdl_cluster(act_quant_kernel<1>, dim3(C, N), dim3(threads_for(bpc)), (unsigned)C, 0, st, gu, ld, I, Kpad,
                                 static_cast<uint8_t*>(bq), ldb, static_cast<uint8_t*>(sfb), g0, static_cast<__half*>(out16));
}

extern "C" int vg_add_rmsnorm_fp4(void* res, const void* delta, const float* w, int N, int h, float eps, int plus_one,
                                  int ld_res, int ld_delta, void* bq, int ldb, void* sfb, float* g0, void* out16,
                                  cudaStream_t st) {
  const int Kpad = ldb * 2;
  if (N < 1 || N > 16 || (ldb % 128) != 0 || Kpad < h || (h % 16) != 0 || (ld_res % 8) != 0 || (ld_delta % 8) != 0 ||
      (Kpad >> 4) > MAX_THREADS * MAXB)
    return -2;
  return (int)launch_pdl(add_rmsnorm_fp4_kernel<0>, dim3(N), dim3(threads_for(Kpad >> 4)), 0, st,
                         static_cast<__nv_bfloat16*>(res), static_cast<const __nv_bfloat16*>(delta), w, h, eps, plus_one,
                         ld_res, ld_delta, Kpad, static_cast<uint8_t*>(bq), ldb, static_cast<uint8_t*>(sfb), g0,
                         static_cast<__half*>(out16), VgCommCtx{});
}

extern "C" int vg_add_rmsnorm_fp4_ar(void* res, const float* w, int N, int h, float eps, int plus_one, int ld_res, void* bq,
                                     int ldb, void* sfb, float* g0, void* out16, const VgCommCtx* ctx, int mode,
                                     cudaStream_t st) {
  const int Kpad = ldb * 2;
  if (!ctx || ctx->world < 2 || N < 1 || N > 16 || (ldb % 128) != 0 || Kpad < h || (h % 16) != 0 || (ld_res % 8) != 0 ||
      (Kpad >> 4) > MAX_THREADS * MAXB)
    return -2;
  if (mode == 2) {
    if (!ctx->mc || (unsigned long long)N * h * 4ull > ctx->mm_slot_bytes) return -5;
    return (int)launch_pdl(add_rmsnorm_fp4_kernel<2>, dim3(N), dim3(threads_for(Kpad >> 4)), 0, st,
                           static_cast<__nv_bfloat16*>(res), (const __nv_bfloat16*)nullptr, w, h, eps, plus_one, ld_res, 0, Kpad,
                           static_cast<uint8_t*>(bq), ldb, static_cast<uint8_t*>(sfb), g0, static_cast<__half*>(out16), *ctx);
  }
  if ((unsigned long long)N * h * 8ull > ctx->slot_bytes) return -5;
  return (int)launch_pdl(add_rmsnorm_fp4_kernel<1>, dim3(N), dim3(threads_for(Kpad >> 4)), 0, st,
                         static_cast<__nv_bfloat16*>(res), (const __nv_bfloat16*)nullptr, w, h, eps, plus_one, ld_res, 0, Kpad,
                         static_cast<uint8_t*>(bq), ldb, static_cast<uint8_t*>(sfb), g0, static_cast<__half*>(out16), *ctx);
}

VG_TRACE_SETTER(vg_trace_set_act_quant)

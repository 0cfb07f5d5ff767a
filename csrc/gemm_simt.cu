// CUDA-core GEMV/GEMM over the canonical (checkpoint-order) weight layouts. One warp per (output row,
// column): K walked in a fixed lane-strided order and reduced with a fixed shuffle tree, every column by
// its own warp (blockIdx.y), so each output column is bit-identical whatever the batch width (the property the reference's
// `gemm_binv_b` provides, reference: kernels/gpu_batch.cu:2385-2403). It serves the tiny bf16 matrices
// (MoE router, shared-expert gate), acts as the on-device cross-check for the tensor-core GEMM, and is
// the fallback when a matrix is too small to tile.
#include "common.cuh"
#include "api.h"

namespace {
using namespace vg;

// Decode 32 consecutive weights of row `m` starting at k0 (k0 % 32 == 0) into fp32.
template <int WFMT>
__device__ __forceinline__ void load_w32(const void* wq, const uint8_t* scales, int m, int K, int k0, float* w) {
  if (WFMT == VG_WF_NVFP4) {
    const uint4 p = *reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(wq) + (size_t)m * (K / 2) + k0 / 2);
    const uint16_t sc = *reinterpret_cast<const uint16_t*>(scales + (size_t)m * (K / 16) + k0 / 16);
    uint32_t s2;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(s2) : "h"(sc));
    const float2 sf = __half22float2(*reinterpret_cast<__half2*>(&s2));
    const uint32_t words[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t h[4];
      asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\tmov.b32 {b0, b1, b2, b3}, %4;\n\t"
          "cvt.rn.f16x2.e2m1x2 %0, b0;\n\tcvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
          "cvt.rn.f16x2.e2m1x2 %2, b2;\n\tcvt.rn.f16x2.e2m1x2 %3, b3;\n\t}\n"
          : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3]) : "r"(words[i]));
      const float s = i < 2 ? sf.x : sf.y;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(*reinterpret_cast<__half2*>(&h[j]));
        w[i * 8 + j * 2] = f.x * s;
        w[i * 8 + j * 2 + 1] = f.y * s;
      }
    }
  } else if (WFMT == VG_WF_FP8) {
    const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(wq) + (size_t)m * K + k0);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const uint4 q = src[i];
      const uint32_t words[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t lo, hi;
        asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(lo) : "h"((uint16_t)(words[j] & 0xffff)));
        asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(hi) : "h"((uint16_t)(words[j] >> 16)));
        const float2 a = __half22float2(*reinterpret_cast<__half2*>(&lo));
        const float2 b = __half22float2(*reinterpret_cast<__half2*>(&hi));
        w[i * 16 + j * 4] = a.x; w[i * 16 + j * 4 + 1] = a.y;
        w[i * 16 + j * 4 + 2] = b.x; w[i * 16 + j * 4 + 3] = b.y;
      }
    }
  } else {
    const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(wq) + (size_t)m * K + k0;
    if ((K & 7) == 0 && (reinterpret_cast<uintptr_t>(wq) & 15) == 0) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 v = reinterpret_cast<const uint4*>(src)[i];
        const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
        for (int j = 0; j < 8; ++j) w[i * 8 + j] = __bfloat162float(b[j]);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) w[i] = __bfloat162float(src[i]);
    }
  }
}

template <int WFMT>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const void* wq, const uint8_t* scales, const float* row_scale,
                                                         const __half* x, void* out, int M, int K, int N, int ldx,
                                                         int ldo, int out_f32) {
  pdl_trigger();
  pdl_wait();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= M) return;
  const int m = warp;
  const int nchunks = K / 32;
  const int tail0 = nchunks * 32;       // K % 32 == 16 leaves one 16-wide tail (NVFP4 blocks are 16 wide)
  {
    const int n = blockIdx.y;
    float acc = 0.0f;
    const __half* xr = x + (size_t)n * ldx;
    for (int c = lane; c < nchunks; c += 32) {
      float w[32];
      load_w32<WFMT>(wq, scales, m, K, c * 32, w);
      const uint4* xv = reinterpret_cast<const uint4*>(xr + c * 32);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 v = xv[i];
        const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __half22float2(h[j]);
          acc = fmaf(w[i * 8 + j * 2], f.x, acc);
          acc = fmaf(w[i * 8 + j * 2 + 1], f.y, acc);
        }
      }
    }
    if (tail0 < K && lane == 0) {
      // scalar tail (at most 16 elements)
      for (int k = tail0; k < K; ++k) {
        float wv;
        if (WFMT == VG_WF_NVFP4) {
          const uint8_t b = static_cast<const uint8_t*>(wq)[(size_t)m * (K / 2) + k / 2];
          const int code = (k & 1) ? (b >> 4) : (b & 0xF);
          const float mag[8] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
          uint32_t s2;
          asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(s2) : "h"((uint16_t)scales[(size_t)m * (K / 16) + k / 16]));
          wv = ((code & 8) ? -mag[code & 7] : mag[code & 7]) * __half22float2(*reinterpret_cast<__half2*>(&s2)).x;
        } else if (WFMT == VG_WF_FP8) {
          uint32_t s2;
          asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(s2) : "h"((uint16_t)static_cast<const uint8_t*>(wq)[(size_t)m * K + k]));
          wv = __half22float2(*reinterpret_cast<__half2*>(&s2)).x;
        } else {
          wv = __bfloat162float(static_cast<const __nv_bfloat16*>(wq)[(size_t)m * K + k]);
        }
        acc = fmaf(wv, __half2float(xr[k]), acc);
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) {
      const float v = acc * (row_scale ? row_scale[m] : 1.0f);
      if (out_f32) static_cast<float*>(out)[(size_t)n * ldo + m] = v;
      else static_cast<__nv_bfloat16*>(out)[(size_t)n * ldo + m] = __float2bfloat16_rn(v);
    }
  }
}

}  // namespace

extern "C" int vg_gemm_simt(const void* wq, const void* scales, const float* row_scale, const void* x_f16, void* out,
                            int out_f32, int M, int K, int N, int ldx, int ldo, int wfmt, cudaStream_t st) {
  if (M <= 0 || N <= 0 || K % 16 != 0) return -2;
  const int threads = 256;
  const dim3 blocks((M * 32 + threads - 1) / threads, N);
  const __half* x = static_cast<const __half*>(x_f16);
  const uint8_t* sc = static_cast<const uint8_t*>(scales);
  switch (wfmt) {
    case VG_WF_NVFP4: launch_pdl(gemm_simt_kernel<VG_WF_NVFP4>, blocks, dim3(threads), 0, st, wq, sc, row_scale, x, out, M, K, N, ldx, ldo, out_f32); break;
    case VG_WF_FP8: launch_pdl(gemm_simt_kernel<VG_WF_FP8>, blocks, dim3(threads), 0, st, wq, sc, row_scale, x, out, M, K, N, ldx, ldo, out_f32); break;
    case VG_WF_BF16: launch_pdl(gemm_simt_kernel<VG_WF_BF16>, blocks, dim3(threads), 0, st, wq, sc, row_scale, x, out, M, K, N, ldx, ldo, out_f32); break;
    default: return -3;
  }
  return (int)cudaGetLastError();
}

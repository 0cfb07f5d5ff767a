// Normalisation, RoPE and small element-wise kernels (one CTA per token column, fp32 math, fixed
// reduction trees so results do not depend on the batch width):
//   vg_add_rmsnorm      residual += delta; normed = rmsnorm(residual) * (1 + w)     -> f16 GEMM input
//   vg_attn_prep        split fused qkv, per-head q/k RMSNorm, partial rotate-half RoPE, KV-cache write
//   vg_swiglu           silu(gate) * up                                            -> f16 GEMM input
//   vg_embed_gather     embedding rows from a bf16 / FP8 / NVFP4 table             -> bf16 residual
//   vg_cast_f16         bf16/f32 -> saturating f16
// They stand in for the reference's rmsnorm_b / fused_res_rmsnorm_b / rmsnorm_perhead_b / rope_b /
// split_qkv_b / split_qgate_b / write_kv_b / silu_mul_b / embed_gather_* (reference:
// kernels/gpu_batch.cu:34-110, :338-405, :821-880, :3011-3100), fused into fewer launches.
#include "common.cuh"
#include "api.h"

namespace {
using namespace vg;

// Vectorised: every thread owns up to MAXC chunks of 8 consecutive elements (16-byte loads/stores), all
// loads are issued before the first use, and the row stays in registers between the two passes.
constexpr int NORM_MAXC = 4;
__global__ void __launch_bounds__(1024) add_rmsnorm_kernel(__nv_bfloat16* res, const __nv_bfloat16* delta, const float* w,
                                                            __half* out16, __nv_bfloat16* out_bf, int h, float eps,
                                                            int plus_one, int ld_res, int ld_delta) {
  pdl_trigger();
  pdl_wait();
  __shared__ float red[32];
  const int n = blockIdx.x;
  __nv_bfloat16* r = res + (size_t)n * ld_res;
  const __nv_bfloat16* d = delta ? delta + (size_t)n * ld_delta : nullptr;
  const int nchunks = h >> 3;
  uint4 rv[NORM_MAXC], dv[NORM_MAXC];
#pragma unroll
  for (int c = 0; c < NORM_MAXC; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch < nchunks) {
      rv[c] = *reinterpret_cast<const uint4*>(r + ch * 8);
      if (d) dv[c] = *reinterpret_cast<const uint4*>(d + ch * 8);
    }
  }
  float v[NORM_MAXC][8];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < NORM_MAXC; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch < nchunks) {
      const __nv_bfloat16* rp = reinterpret_cast<const __nv_bfloat16*>(&rv[c]);
      const __nv_bfloat16* dp = reinterpret_cast<const __nv_bfloat16*>(&dv[c]);
      uint4 upd;
      __nv_bfloat16* up = reinterpret_cast<__nv_bfloat16*>(&upd);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float x = __bfloat162float(rp[i]);
        if (d) {
          x += __bfloat162float(dp[i]);
          up[i] = __float2bfloat16_rn(x);
          x = __bfloat162float(up[i]);
        }
        v[c][i] = x;
        ss += x * x;
      }
      if (d) *reinterpret_cast<uint4*>(r + ch * 8) = upd;
    }
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)h + eps);
#pragma unroll
  for (int c = 0; c < NORM_MAXC; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch < nchunks) {
      const float4 w0 = *reinterpret_cast<const float4*>(w + ch * 8);
      const float4 w1 = *reinterpret_cast<const float4*>(w + ch * 8 + 4);
      const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
      uint4 o16, obf;
      __half* hp = reinterpret_cast<__half*>(&o16);
      __nv_bfloat16* bp = reinterpret_cast<__nv_bfloat16*>(&obf);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float y = v[c][i] * inv * (plus_one ? 1.0f + ww[i] : ww[i]);
        hp[i] = f32_to_f16_sat(y);
        bp[i] = __float2bfloat16_rn(y);
      }
      if (out16) *reinterpret_cast<uint4*>(out16 + (size_t)n * h + ch * 8) = o16;
      if (out_bf) *reinterpret_cast<uint4*>(out_bf + (size_t)n * h + ch * 8) = obf;
    }
  }
}

// One CTA per (column, head slot). Head slots: [0, nh) query heads, [nh, nh+nkv) key heads,
// [nh+nkv, nh+2nkv) value heads. blockDim.x == hd.
// 4-bit cache write: sixteen consecutive dims share one f16 scale (amax / 7), codes are round(v / scale) + 8.
VG_DEVINL void kv_q4_store(float v, int d, uint8_t* codes_row, __half* scale_row) {
  float amax = fabsf(v);
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const __half sc = __float2half_rn(amax / 7.0f);
  const float scf = __half2float(sc);
  const float inv = scf > 0.f ? 1.0f / scf : 0.f;
  const int code = (int)fminf(fmaxf(rintf(v * inv), -7.0f), 7.0f) + 8;
  const int hi = __shfl_xor_sync(0xffffffffu, code, 1);
  if ((d & 1) == 0) codes_row[d >> 1] = (uint8_t)(code | (hi << 4));
  if ((d & 15) == 0) scale_row[d >> 4] = sc;
}

__global__ void attn_prep_kernel(const __nv_bfloat16* qkv, int ld_qkv, const float* q_norm, const float* k_norm,
                                 const int* pos, const int* slot, const int* kv_row, __nv_bfloat16* q_out,
                                 __nv_bfloat16* kc, __nv_bfloat16* vc, int nh, int nkv, int hd, int rdim, int max_seq,
                                 float eps, float log2_theta, int gated, __half* k_scale, __half* v_scale) {
  pdl_trigger();
  pdl_wait();
  __shared__ float red[32];
  extern __shared__ float xs[];
  const int n = blockIdx.x, hs = blockIdx.y, d = threadIdx.x;
  const int qw = gated ? 2 * hd : hd;
  const __nv_bfloat16* src;
  const float* nw = nullptr;
  if (hs < nh) { src = qkv + (size_t)n * ld_qkv + hs * qw; nw = q_norm; }
  else if (hs < nh + nkv) { src = qkv + (size_t)n * ld_qkv + nh * qw + (hs - nh) * hd; nw = k_norm; }
  else { src = qkv + (size_t)n * ld_qkv + nh * qw + nkv * hd + (hs - nh - nkv) * hd; }
  float v = __bfloat162float(src[d]);
  if (hs >= nh + nkv) {
    const int s = slot[n], row = kv_row[n];
    const size_t r = ((size_t)s * nkv + (hs - nh - nkv)) * max_seq + row;
    if (v_scale) kv_q4_store(v, d, reinterpret_cast<uint8_t*>(vc) + r * (hd / 2), v_scale + r * (hd / 16));
    else vc[r * hd + d] = __float2bfloat16_rn(v);
    return;
  }
  float ss = block_sum(v * v, red);
  v = v * rsqrtf(ss / (float)hd + eps) * (1.0f + nw[d]);
  xs[d] = v;
  __syncthreads();
  if (d < rdim) {
    const int half = rdim / 2;
    const int i = d < half ? d : d - half;
    // inv_freq = theta^(-2i/rdim)
    const float inv_freq = exp2f(-log2_theta * (2.0f * (float)i / (float)rdim));
    float sn, cs;
    sincosf((float)pos[n] * inv_freq, &sn, &cs);
    const float x1 = xs[i], x2 = xs[i + half];
    v = d < half ? x1 * cs - x2 * sn : x2 * cs + x1 * sn;
  }
  if (hs < nh) {
    q_out[((size_t)n * nh + hs) * hd + d] = __float2bfloat16_rn(v);
  } else {
    const int s = slot[n], row = kv_row[n];
    const size_t r = ((size_t)s * nkv + (hs - nh)) * max_seq + row;
    if (k_scale) kv_q4_store(v, d, reinterpret_cast<uint8_t*>(kc) + r * (hd / 2), k_scale + r * (hd / 16));
    else kc[r * hd + d] = __float2bfloat16_rn(v);
  }
}

__global__ void swiglu_kernel(const __nv_bfloat16* gu, __half* out, int I, int ld, size_t total) {
  pdl_trigger();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t n = i / I, c = i % I;
  const float g = __bfloat162float(gu[n * ld + c]);
  const float u = __bfloat162float(gu[n * ld + I + c]);
  out[i] = f32_to_f16_sat(silu(g) * u);
}

// eight elements per thread (16-byte loads / stores): the form prefill widths use
__global__ void swiglu_vec8_kernel(const __nv_bfloat16* __restrict__ gu, __half* __restrict__ out, int I8, int ld, size_t total8) {
  pdl_trigger();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total8) return;
  const size_t n = i / I8, c = (i % I8) * 8;
  const uint4 g4 = *reinterpret_cast<const uint4*>(gu + n * ld + c);
  const uint4 u4 = *reinterpret_cast<const uint4*>(gu + n * ld + (size_t)I8 * 8 + c);
  const __nv_bfloat16* g = reinterpret_cast<const __nv_bfloat16*>(&g4);
  const __nv_bfloat16* u = reinterpret_cast<const __nv_bfloat16*>(&u4);
  uint4 o4;
  __half* o = reinterpret_cast<__half*>(&o4);
#pragma unroll
  for (int k = 0; k < 8; ++k) o[k] = f32_to_f16_sat(silu(__bfloat162float(g[k])) * __bfloat162float(u[k]));
  *reinterpret_cast<uint4*>(out + n * (size_t)I8 * 8 + c) = o4;
}

template <typename T>
__global__ void cast_f16_kernel(const T* in, __half* out, size_t total) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < total) out[i] = f32_to_f16_sat((float)in[i]);
}

__global__ void embed_gather_kernel(const void* table, const uint8_t* scales, const float* row_scale, const int* tok,
                                    __nv_bfloat16* out, int h, int wfmt) {
  pdl_trigger();
  pdl_wait();
  const int n = blockIdx.x;
  const size_t t = (size_t)tok[n];
  for (int i = threadIdx.x; i < h; i += blockDim.x) {
    float v;
    if (wfmt == VG_WF_BF16) {
      v = __bfloat162float(static_cast<const __nv_bfloat16*>(table)[t * h + i]);
    } else if (wfmt == VG_WF_FP8) {
      uint32_t s2;
      asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(s2) : "h"((uint16_t)static_cast<const uint8_t*>(table)[t * h + i]));
      v = __half22float2(*reinterpret_cast<__half2*>(&s2)).x * row_scale[t];
    } else {
      const uint8_t b = static_cast<const uint8_t*>(table)[t * (h / 2) + i / 2];
      const int code = (i & 1) ? (b >> 4) : (b & 0xF);
      const float mag = (code & 4) ? ((code & 2) ? ((code & 1) ? 6.f : 4.f) : ((code & 1) ? 3.f : 2.f))
                                   : ((code & 2) ? ((code & 1) ? 1.5f : 1.f) : ((code & 1) ? .5f : 0.f));
      uint32_t s2;
      asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(s2) : "h"((uint16_t)scales[t * (h / 16) + i / 16]));
      // value = code * (block scale * tensor scale), the order the canonical dequantisation uses.
      v = ((code & 8) ? -mag : mag) * (__half22float2(*reinterpret_cast<__half2*>(&s2)).x * row_scale[t]);
    }
    out[(size_t)n * h + i] = __float2bfloat16_rn(v);
  }
}

}  // namespace

extern "C" int vg_add_rmsnorm(void* res, const void* delta, const float* w, void* out_f16, void* out_bf16, int N, int h,
                              float eps, int plus_one, int ld_res, int ld_delta, cudaStream_t st) {
  if (N <= 0) return 0;
  if ((h & 7) || (ld_res & 7) || (ld_delta & 7) || h > 8 * 1024 * NORM_MAXC) return -2;
  int threads = ((h >> 3) + 31) / 32 * 32;
  if (threads > 1024) threads = ((((h >> 3) + NORM_MAXC - 1) / NORM_MAXC) + 31) / 32 * 32;
  launch_pdl(add_rmsnorm_kernel, dim3(N), dim3(threads), 0, st, static_cast<__nv_bfloat16*>(res),
                                                       static_cast<const __nv_bfloat16*>(delta), w,
                                                       static_cast<__half*>(out_f16),
                                                       static_cast<__nv_bfloat16*>(out_bf16), h, eps, plus_one, ld_res,
                                                       ld_delta);
  return (int)cudaGetLastError();
}

extern "C" int vg_attn_prep(const void* qkv, int ld_qkv, const float* q_norm, const float* k_norm, const int* pos,
                            const int* slot, const int* kv_row, void* q_out, void* kc, void* vc, int N, int nh, int nkv,
                            int hd, int rdim, int max_seq, float eps, float theta, int gated, void* k_scale, void* v_scale,
                            cudaStream_t st) {
  if (N <= 0) return 0;
  if (hd > 1024 || (hd & 31) || ((k_scale == nullptr) != (v_scale == nullptr))) return -2;
  dim3 grid(N, nh + 2 * nkv);
  launch_pdl(attn_prep_kernel, dim3(grid), dim3(hd), hd * sizeof(float), st, 
      static_cast<const __nv_bfloat16*>(qkv), ld_qkv, q_norm, k_norm, pos, slot, kv_row,
      static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(kc), static_cast<__nv_bfloat16*>(vc), nh, nkv, hd,
      rdim, max_seq, eps, log2f(theta), gated, static_cast<__half*>(k_scale), static_cast<__half*>(v_scale));
  return (int)cudaGetLastError();
}

extern "C" int vg_swiglu(const void* gu, void* out_f16, int N, int I, int ld, cudaStream_t st) {
  const size_t total = (size_t)N * I;
  if (!total) return 0;
  if (I % 8 == 0 && ld % 8 == 0 && ((reinterpret_cast<uintptr_t>(gu) | reinterpret_cast<uintptr_t>(out_f16)) & 15) == 0) {
    const size_t total8 = total / 8;
    launch_pdl(swiglu_vec8_kernel, dim3((unsigned)((total8 + 255) / 256)), dim3(256), 0, st, static_cast<const __nv_bfloat16*>(gu),
               static_cast<__half*>(out_f16), I / 8, ld, total8);
    return (int)cudaGetLastError();
  }
  launch_pdl(swiglu_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, st, static_cast<const __nv_bfloat16*>(gu),
                                                                 static_cast<__half*>(out_f16), I, ld, total);
  return (int)cudaGetLastError();
}

extern "C" int vg_cast_f16(const void* in, int in_is_f32, void* out_f16, long long total, cudaStream_t st) {
  if (total <= 0) return 0;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (in_is_f32) cast_f16_kernel<float><<<blocks, 256, 0, st>>>(static_cast<const float*>(in), static_cast<__half*>(out_f16), (size_t)total);
  else cast_f16_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(in), static_cast<__half*>(out_f16), (size_t)total);
  return (int)cudaGetLastError();
}

extern "C" int vg_embed_gather(const void* table, const void* scales, const float* row_scale, const int* tok, void* out,
                               int N, int h, int wfmt, cudaStream_t st) {
  if (N <= 0) return 0;
  launch_pdl(embed_gather_kernel, dim3(N), dim3(256), 0, st, table, static_cast<const uint8_t*>(scales), row_scale, tok,
                                         static_cast<__nv_bfloat16*>(out), h, wfmt);
  return (int)cudaGetLastError();
}

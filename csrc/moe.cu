// Mixture-of-experts support kernels around the grouped tensor-core GEMM:
//   vg_moe_router     top-k selection + combine weights from fp32 router logits; also emits the per-pair
//                     group table (expert rebased to this rank's resident band, -1 when not resident)
//   vg_moe_sort       counting sort of (token, slot) pairs by expert: counts, offsets, work-item tile map,
//                     permutation - entirely on the device (no host read-back of the offsets, unlike the
//                     reference at src/gpu.rs:2323-2325)
//   vg_moe_gather     activation rows permuted into expert order for the prefill grouped GEMM
//   vg_moe_combine    weighted sum of a token's expert outputs in slot order (+ gated shared expert)
// Router math (reference: kernels/gpu_batch.cu:3102-3240): softmax flavour selects the top-k logits (lowest
// index wins ties) and weights them exp(l - max) / sum over the selected k; sigmoid flavour selects by
// sigmoid(l) + bias and weights by the unbiased sigmoid, renormalised and scaled. The combine adds slots in
// slot order, so the result does not depend on the (atomic) order pairs were scattered in.
#include "common.cuh"
#include "api.h"

namespace {
using namespace vg;

constexpr int MAX_E = 1024;
constexpr int MAX_K = 16;

// One warp per token: the E scores live in registers (E / 32 per lane), each of the K rounds is a local
// arg-max plus a shuffle arg-max (ties to the lower expert index), no block barriers.
template <int PER>
__global__ void __launch_bounds__(32) router_kernel(const float* __restrict__ logits, int E, int K, int sigmoid_mode,
                                                     const float* __restrict__ bias, int norm, float scaling, int e_base,
                                                     int n_local, int* __restrict__ ids, float* __restrict__ wts,
                                                     int* __restrict__ g_exp, int* __restrict__ g_off, int* __restrict__ g_cnt) {
  pdl_trigger();
  pdl_wait();
  const int n = blockIdx.x, lane = threadIdx.x;
  float score[PER], raw[PER];
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int e = j * 32 + lane;
    score[j] = -INFINITY; raw[j] = 0.f;
    if (e < E) {
      const float l = logits[(size_t)n * E + e];
      const float sv = sigmoid_mode ? sigmoidf(l) : l;
      raw[j] = sv;
      score[j] = sigmoid_mode && bias ? sv + bias[e] : sv;
    }
  }
  float selv[MAX_K];
  int seli[MAX_K];
#pragma unroll 1
  for (int r = 0; r < K; ++r) {
    float v = -INFINITY, rv = 0.f;
    int idx = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int e = j * 32 + lane;
      if (score[j] > v || (score[j] == v && e < idx)) { v = score[j]; idx = e; rv = raw[j]; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      const float orv = __shfl_xor_sync(0xffffffffu, rv, o);
      if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; rv = orv; }
    }
    selv[r] = rv;
    seli[r] = idx;
#pragma unroll
    for (int j = 0; j < PER; ++j)
      if (j * 32 + lane == idx) score[j] = -INFINITY;
  }
  if (lane == 0) {
    float w[MAX_K];
    if (sigmoid_mode) {
      float sum = 0.f;
      for (int r = 0; r < K; ++r) { w[r] = selv[r]; sum += w[r]; }
      for (int r = 0; r < K; ++r) w[r] = (norm ? w[r] / sum : w[r]) * scaling;
    } else {
      const float mx = selv[0];
      float sum = 0.f;
      for (int r = 0; r < K; ++r) { w[r] = __expf(selv[r] - mx); sum += w[r]; }
      for (int r = 0; r < K; ++r) w[r] /= sum;
    }
    for (int r = 0; r < K; ++r) {
      const int p = n * K + r;
      ids[p] = seli[r];
      wts[p] = w[r];
      const int loc = seli[r] - e_base;
      if (g_exp) { g_exp[p] = (loc >= 0 && loc < n_local) ? loc : -1; g_off[p] = p; g_cnt[p] = 1; }
    }
  }
}

__global__ void moe_count_kernel(const int* __restrict__ ids, int P, int e_base, int n_local, int* __restrict__ cnt) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= P) return;
  const int loc = ids[p] - e_base;
  if (loc >= 0 && loc < n_local) atomicAdd(&cnt[loc], 1);
}

// One block: exclusive scan of the counts -> offsets and cursors, group table, tile map, item count.
__global__ void __launch_bounds__(1024) moe_scan_kernel(int* __restrict__ cnt, int n_local, int bn, int* __restrict__ g_exp,
                                                         int* __restrict__ g_off, int* __restrict__ g_cnt,
                                                         int* __restrict__ cursor, int* __restrict__ tilemap,
                                                         int* __restrict__ n_items) {
  __shared__ int off[MAX_E + 1], toff[MAX_E + 1];
  if (threadIdx.x == 0) {
    int o = 0, t = 0;
    for (int e = 0; e < n_local; ++e) {
      off[e] = o; toff[e] = t;
      o += cnt[e];
      t += (cnt[e] + bn - 1) / bn;
    }
    off[n_local] = o; toff[n_local] = t;
    *n_items = t;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < n_local; e += blockDim.x) {
    g_exp[e] = e; g_off[e] = off[e]; g_cnt[e] = cnt[e]; cursor[e] = off[e];
    for (int t = toff[e]; t < toff[e + 1]; ++t) { tilemap[2 * t] = e; tilemap[2 * t + 1] = t - toff[e]; }
  }
}

__global__ void moe_scatter_kernel(const int* __restrict__ ids, int P, int e_base, int n_local, int* __restrict__ cursor,
                                   int* __restrict__ perm, int* __restrict__ inv) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= P) return;
  const int loc = ids[p] - e_base;
  if (loc >= 0 && loc < n_local) {
    const int pos = atomicAdd(&cursor[loc], 1);
    perm[pos] = p;
    inv[p] = pos;
  } else {
    inv[p] = -1;
  }
}

__global__ void moe_gather_kernel(const __half* __restrict__ x, int ldx, const int* __restrict__ perm, const int* __restrict__ total,
                                  int topk, int h, __half* __restrict__ out) {
  const int pos = blockIdx.x;
  if (pos >= *total) return;
  const int tok = perm[pos] / topk;
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)tok * ldx);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)pos * h);
  for (int i = threadIdx.x; i < h / 8; i += blockDim.x) dst[i] = src[i];
}

__global__ void moe_total_kernel(const int* __restrict__ g_off, const int* __restrict__ g_cnt, int n_local, int* __restrict__ total) {
  if (threadIdx.x == 0 && blockIdx.x == 0) *total = n_local > 0 ? g_off[n_local - 1] + g_cnt[n_local - 1] : 0;
}

// out[t, :] = sum_slot w[t, slot] * y[inv[t*K + slot], :]   (slot order; non-resident pairs contribute 0)
//           (+ gate[t] * shared[t, :] when a shared expert is given)
// out[t] = sum_s wts[t, s] * y[inv[t, s]] (slot order) + sigmoid(gate) * shared[t]; eight columns per thread,
// all expert rows of a thread's columns are in flight before the first add.
// PUSH (expert parallelism at decode widths): the row is this rank's partial sum over its resident experts. It is
// not stored but sent, as fp32 (value, epoch) pairs, into the receive slot of every rank (this one included), where
// the residual-add / RMSNorm kernel that follows polls its own memory and sums the ranks in order: combine and
// all-reduce in one kernel, no barrier and no separate reduction launch. The caller passes the replicated shared
// expert on one rank only.
template <bool PUSH>
__global__ void __launch_bounds__(256) moe_combine_kernel(const __nv_bfloat16* __restrict__ y, int ldy,
                                                           const int* __restrict__ inv, const float* __restrict__ wts, int topk,
                                                           const __nv_bfloat16* __restrict__ shared,
                                                           const float* __restrict__ gate_logit, __nv_bfloat16* __restrict__ out,
                                                           int h, const VgCommCtx c) {
  __shared__ int spos[MAX_K];
  __shared__ float sw[MAX_K];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  if (threadIdx.x < topk) {
    spos[threadIdx.x] = inv ? inv[t * topk + threadIdx.x] : t * topk + threadIdx.x;
    sw[threadIdx.x] = wts[t * topk + threadIdx.x];
  }
  __syncthreads();
  const float g = gate_logit ? sigmoidf(gate_logit[t]) : 1.0f;
  const uint32_t e = PUSH ? *c.epoch + 1 : 0;   // (read after the wait: the preceding collective's consumer bumps it)
  for (int i = threadIdx.x * 8; i < h; i += blockDim.x * 8) {
    uint4 rows[MAX_K];
#pragma unroll
    for (int s = 0; s < MAX_K; ++s)
      if (s < topk && spos[s] >= 0) rows[s] = *reinterpret_cast<const uint4*>(y + (size_t)spos[s] * ldy + i);
    uint4 sh = make_uint4(0, 0, 0, 0);
    if (shared) sh = *reinterpret_cast<const uint4*>(shared + (size_t)t * h + i);
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.f;
#pragma unroll
    for (int s = 0; s < MAX_K; ++s) {
      if (s < topk && spos[s] >= 0) {
        const __nv_bfloat16* r = reinterpret_cast<const __nv_bfloat16*>(&rows[s]);
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] += sw[s] * __bfloat162float(r[k]);
      }
    }
    uint4 o4;
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(&o4);
    const __nv_bfloat16* shb = reinterpret_cast<const __nv_bfloat16*>(&sh);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (shared) acc[k] += g * __bfloat162float(shb[k]);
      o[k] = __float2bfloat16_rn(acc[k]);
    }
    if (PUSH) {
      for (int q = 0; q < c.world; ++q) {
        const int peer = (c.rank + q) % c.world;
        uint2* dst = reinterpret_cast<uint2*>(c.data[peer] + c.slots_off + (size_t)((e & 1) * MAX_RANKS + c.rank) * c.slot_bytes) +
                     ((size_t)t * h + i);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(dst + k), "r"(__float_as_uint(acc[k])), "r"(e) : "memory");
      }
    } else {
      *reinterpret_cast<uint4*>(out + (size_t)t * h + i) = o4;
    }
  }
}

__global__ void moe_add_shared_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ shared,
                                      const float* __restrict__ gate_logit, int h, size_t total) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int t = (int)(i / h);
  const float g = gate_logit ? sigmoidf(gate_logit[t]) : 1.0f;
  out[i] = __float2bfloat16_rn(__bfloat162float(out[i]) + g * __bfloat162float(shared[i]));
}

}  // namespace

extern "C" int vg_moe_router(const float* logits, int N, int E, int K, int sigmoid_mode, const float* bias, int norm,
                             float scaling, int e_base, int n_local, int* ids, float* wts, int* g_exp, int* g_off,
                             int* g_cnt, cudaStream_t st) {
  if (N <= 0) return 0;
  if (E > MAX_E || K > MAX_K || K > E) return -2;
  if (E <= 256)
    launch_pdl(router_kernel<8>, dim3(N), dim3(32), 0, st, logits, E, K, sigmoid_mode, bias, norm, scaling, e_base, n_local, ids,
               wts, g_exp, g_off, g_cnt);
  else
    launch_pdl(router_kernel<MAX_E / 32>, dim3(N), dim3(32), 0, st, logits, E, K, sigmoid_mode, bias, norm, scaling, e_base,
               n_local, ids, wts, g_exp, g_off, g_cnt);
  return (int)cudaGetLastError();
}

// Prefill-side sort. cnt/cursor: [n_local] scratch; perm/inv: [P]; tilemap: [max_items][2]; total: [1].
extern "C" int vg_moe_sort(const int* ids, int P, int e_base, int n_local, int bn, int* cnt, int* cursor, int* g_exp,
                           int* g_off, int* g_cnt, int* tilemap, int* n_items, int* perm, int* inv, int* total,
                           cudaStream_t st) {
  if (P <= 0) return 0;
  if (n_local > MAX_E) return -2;
  cudaMemsetAsync(cnt, 0, sizeof(int) * n_local, st);
  moe_count_kernel<<<(P + 255) / 256, 256, 0, st>>>(ids, P, e_base, n_local, cnt);
  moe_scan_kernel<<<1, 1024, 0, st>>>(cnt, n_local, bn, g_exp, g_off, g_cnt, cursor, tilemap, n_items);
  moe_scatter_kernel<<<(P + 255) / 256, 256, 0, st>>>(ids, P, e_base, n_local, cursor, perm, inv);
  moe_total_kernel<<<1, 32, 0, st>>>(g_off, g_cnt, n_local, total);
  return (int)cudaGetLastError();
}

extern "C" int vg_moe_gather(const void* x_f16, int ldx, const int* perm, const int* total, int max_rows, int topk, int h,
                             void* out_f16, cudaStream_t st) {
  if (max_rows <= 0) return 0;
  if (h % 8) return -2;
  moe_gather_kernel<<<max_rows, 128, 0, st>>>(static_cast<const __half*>(x_f16), ldx, perm, total, topk, h,
                                               static_cast<__half*>(out_f16));
  return (int)cudaGetLastError();
}

extern "C" int vg_moe_combine(const void* y, int ldy, const int* inv, const float* wts, int N, int topk, const void* shared,
                              const float* gate_logit, void* out, int h, cudaStream_t st) {
  if (N <= 0) return 0;
  if (topk > MAX_K || (h % 8) != 0 || (ldy % 8) != 0) return -2;
  launch_pdl(moe_combine_kernel<false>, dim3(N), dim3(256), 0, st, static_cast<const __nv_bfloat16*>(y), ldy, inv, wts, topk,
             static_cast<const __nv_bfloat16*>(shared), gate_logit, static_cast<__nv_bfloat16*>(out), h, VgCommCtx{});
  return (int)cudaGetLastError();
}

// Combine fused with the expert-parallel all-reduce (push half): see moe_combine_kernel<true>. The consumer is
// vg_add_rmsnorm_fp4_ar on every rank; `shared` / `gate_logit` are passed on one rank only.
extern "C" int vg_moe_combine_push(const void* y, int ldy, const int* inv, const float* wts, int N, int topk, const void* shared,
                                   const float* gate_logit, int h, const VgCommCtx* ctx, cudaStream_t st) {
  if (N <= 0) return 0;
  if (!ctx || topk > MAX_K || (h % 16) != 0 || (ldy % 8) != 0) return -2;
  if (ctx->world < 1 || ctx->world > MAX_RANKS || (unsigned long long)N * h * 8ull > ctx->slot_bytes) return -2;
  launch_pdl(moe_combine_kernel<true>, dim3(N), dim3(256), 0, st, static_cast<const __nv_bfloat16*>(y), ldy, inv, wts, topk,
             static_cast<const __nv_bfloat16*>(shared), gate_logit, static_cast<__nv_bfloat16*>(nullptr), h, *ctx);
  return (int)cudaGetLastError();
}

extern "C" int vg_moe_add_shared(void* out, const void* shared, const float* gate_logit, int N, int h, cudaStream_t st) {
  const size_t total = (size_t)N * h;
  if (!total) return 0;
  moe_add_shared_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(static_cast<__nv_bfloat16*>(out),
                                                                         static_cast<const __nv_bfloat16*>(shared),
                                                                         gate_logit, h, total);
  return (int)cudaGetLastError();
}

// Sampling tail on fp32 logits [N, V]: penalties, argmax, nucleus construction and draw, per-position NLL.
// Numeric contract (reference: kernels/gpu_batch.cu:877-903, :930-990, :2206-2272, :2602-2640):
//   * penalties over a per-lane list of (token, count): repetition divides positive logits and
//     multiplies negative ones, presence subtracts a flat amount, frequency subtracts amount * count;
//   * greedy when temperature < 1e-6; top-k clamped to [1, 64], selected by repeated arg-max with the
//     lowest index winning ties; softmax over the scaled top-k; nucleus = smallest prefix whose mass
//     reaches top_p * total; draw with the LCG s = s*1664525 + 1013904223, u = (s >> 8) / 2^24 scaled by
//     the nucleus mass.
// The arg-max selection never modifies the logits: round r picks the largest element that is strictly
// after the previous pick in (value descending, index ascending) order.
#include "common.cuh"
#include "api.h"

namespace {
using namespace vg;

constexpr int MAXK = 64;

struct Best { float v; int i; };
__device__ __forceinline__ bool better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

__device__ __forceinline__ Best block_best(Best b, Best* sm) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, b.v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, b.i, o);
    if (better(ov, oi, b.v, b.i)) { b.v = ov; b.i = oi; }
  }
  __syncthreads();
  if (lane == 0) sm[w] = b;
  __syncthreads();
  Best r = lane < nw ? sm[lane] : Best{-INFINITY, 0x7fffffff};
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, r.v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, r.i, o);
    if (better(ov, oi, r.v, r.i)) { r.v = ov; r.i = oi; }
  }
  return r;
}

__global__ void __launch_bounds__(1024) argmax_kernel(const float* logits, int V, int ld, int* out, float* out_val,
                                                       int idx_offset) {
  pdl_trigger();
  pdl_wait();
  __shared__ Best sm[32];
  const float* row = logits + (size_t)blockIdx.x * ld;
  Best b{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = row[i];
    if (better(v, i, b.v, b.i)) { b.v = v; b.i = i; }
  }
  b = block_best(b, sm);
  if (threadIdx.x == 0) {
    out[blockIdx.x] = b.i + idx_offset;
    if (out_val) out_val[blockIdx.x] = b.v;
  }
}

__global__ void penalty_kernel(float* logits, int ld, const int* toks, const int* counts, const int* n_toks, int max_toks,
                               const float* rep, const float* pres, const float* freq, int V) {
  const int n = blockIdx.x;
  const int cnt = n_toks[n];
  const float r = rep[n], p = pres[n], f = freq[n];
  for (int i = threadIdx.x; i < cnt; i += blockDim.x) {
    const int t = toks[n * max_toks + i];
    if (t < 0 || t >= V) continue;
    float v = logits[(size_t)n * ld + t];
    if (r != 1.0f) v = v > 0.f ? v / r : v * r;
    v -= p + f * (float)counts[n * max_toks + i];
    logits[(size_t)n * ld + t] = v;
  }
}

// Nucleus for one column: ids/probs of the kept tokens (probabilities of the scaled top-k softmax, not
// renormalised to the nucleus), their count, and optionally a drawn token.
__global__ void __launch_bounds__(256) nucleus_kernel(const float* logits, int V, int ld, const float* temp,
                                                       const int* top_k, const float* top_p, const unsigned* seed,
                                                       int* out_tok, int* ids, float* probs, int* n_keep) {
  __shared__ Best sm[32];
  __shared__ float sv[MAXK];
  __shared__ int si[MAXK];
  const int n = blockIdx.x;
  const float* row = logits + (size_t)n * ld;
  const float T = temp[n];
  int K = top_k[n];
  K = K < 1 ? 1 : (K > MAXK ? MAXK : K);
  if (T < 1e-6f) K = 1;
  float pv = INFINITY;
  int pi = -1;
  for (int r = 0; r < K; ++r) {
    Best b{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float v = row[i];
      const bool after = v < pv || (v == pv && i > pi);
      if (after && better(v, i, b.v, b.i)) { b.v = v; b.i = i; }
    }
    b = block_best(b, sm);
    if (threadIdx.x == 0) { sv[r] = b.v; si[r] = b.i; }
    pv = b.v; pi = b.i;
    if (b.i == 0x7fffffff) { K = r; break; }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int keep = 1;
    int tok = si[0];
    if (T >= 1e-6f && K > 0) {
      const float mx = sv[0] / T;
      float sum = 0.f;
      for (int r = 0; r < K; ++r) { sv[r] = __expf(sv[r] / T - mx); sum += sv[r]; }
      for (int r = 0; r < K; ++r) sv[r] /= sum;
      const float target = top_p[n];
      float cum = 0.f;
      keep = K;
      for (int r = 0; r < K; ++r) { cum += sv[r]; if (cum >= target) { keep = r + 1; break; } }
      float mass = 0.f;
      for (int r = 0; r < keep; ++r) mass += sv[r];
      if (out_tok) {
        unsigned s = seed[n] * 1664525u + 1013904223u;
        const float u = (float)(s >> 8) * (1.0f / 16777216.0f) * mass;
        float c = 0.f;
        tok = si[keep - 1];
        for (int r = 0; r < keep; ++r) { c += sv[r]; if (u < c) { tok = si[r]; break; } }
      }
    } else {
      sv[0] = 1.0f;
    }
    if (out_tok) out_tok[n] = tok;
    if (n_keep) n_keep[n] = keep;
    if (ids) for (int r = 0; r < keep; ++r) { ids[n * MAXK + r] = si[r]; probs[n * MAXK + r] = sv[r]; }
  }
}

__global__ void __launch_bounds__(1024) nll_kernel(const float* logits, int V, int ld, const int* target, float* out) {
  __shared__ float red[32];
  const float* row = logits + (size_t)blockIdx.x * ld;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, row[i]);
  mx = warp_max(mx);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = (threadIdx.x & 31) < (blockDim.x >> 5) ? red[threadIdx.x & 31] : -INFINITY;
  mx = warp_max(mx);
  float s = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) s += __expf(row[i] - mx);
  s = block_sum(s, red);
  if (threadIdx.x == 0) out[blockIdx.x] = (mx + logf(s)) - row[target[blockIdx.x]];
}

}  // namespace

extern "C" int vg_argmax(const float* logits, int N, int V, int ld, int* out, float* out_val, int idx_offset,
                         cudaStream_t st) {
  if (N <= 0) return 0;
  launch_pdl(argmax_kernel, dim3(N), dim3(1024), 0, st, logits, V, ld, out, out_val, idx_offset);
  return (int)cudaGetLastError();
}

extern "C" int vg_penalty(float* logits, int N, int V, int ld, const int* toks, const int* counts, const int* n_toks,
                          int max_toks, const float* rep, const float* pres, const float* freq, cudaStream_t st) {
  if (N <= 0) return 0;
  penalty_kernel<<<N, 64, 0, st>>>(logits, ld, toks, counts, n_toks, max_toks, rep, pres, freq, V);
  return (int)cudaGetLastError();
}

extern "C" int vg_nucleus(const float* logits, int N, int V, int ld, const float* temp, const int* top_k,
                          const float* top_p, const unsigned* seed, int* out_tok, int* ids, float* probs, int* n_keep,
                          cudaStream_t st) {
  if (N <= 0) return 0;
  nucleus_kernel<<<N, 256, 0, st>>>(logits, V, ld, temp, top_k, top_p, seed, out_tok, ids, probs, n_keep);
  return (int)cudaGetLastError();
}

extern "C" int vg_nll(const float* logits, int N, int V, int ld, const int* target, float* out, cudaStream_t st) {
  if (N <= 0) return 0;
  nll_kernel<<<N, 1024, 0, st>>>(logits, V, ld, target, out);
  return (int)cudaGetLastError();
}

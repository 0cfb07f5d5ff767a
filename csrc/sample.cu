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
                               const float* rep, const float* pres, const float* freq, int V, int idx_offset) {
  pdl_trigger();
  pdl_wait();
  const int n = blockIdx.x;
  const int cnt = n_toks[n];
  const float r = rep[n], p = pres[n], f = freq[n];
  for (int i = threadIdx.x; i < cnt; i += blockDim.x) {
    const int t = toks[n * max_toks + i] - idx_offset;      // ids outside this rank's vocabulary shard are skipped
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


// ------------------------------------------------------------------ chunked top-k / nucleus / speculative verify
// Token selection in three small launches that also work on a vocabulary-sharded head:
//   topk_chunk_kernel   grid (row, chunk): the chunk's top-K in (value desc, index asc) order, found in shared memory;
//   topk_merge_kernel   one CTA per row: merges `n_lists` sorted K-lists (this rank's chunks, or every rank's local
//                       top-K after the small all-gather) into the row's top-K; in `finish` mode it goes on to the
//                       softmax over the scaled top-K, the top-p cut and the draw, which every rank computes alike;
//   spec_verify_kernel  accept / residual-resample / bonus over one lane's verify columns from their nuclei.
// Uniforms come from the host's keyed generator, so a request's stream of draws does not depend on which path
// (host or device) selected its tokens. Probabilities are fp32; masses, cumulative sums and the accept test use
// double in the same order as the host implementation, so both make the same decisions.
constexpr int TOPK_CHUNK = 4096;

struct Cand { float v; int i; };

__device__ __forceinline__ int clamp_k(int k, float T) {
  k = k < 1 ? 1 : (k > MAXK ? MAXK : k);
  return T < 1e-6f ? 1 : k;
}

// K rounds of "largest element strictly after the previous pick" over `n` candidates in shared memory.
__device__ __forceinline__ int select_topk(const float* cv, const int* ci, int n, int K, Best* sm, float* ov, int* oi) {
  float pv = INFINITY;
  int pi = -1;
  int got = 0;
  for (int r = 0; r < K; ++r) {
    Best b{-INFINITY, 0x7fffffff};
    for (int j = threadIdx.x; j < n; j += blockDim.x) {
      const float v = cv[j];
      const int i = ci[j];
      const bool after = v < pv || (v == pv && i > pi);
      if (after && i != 0x7fffffff && better(v, i, b.v, b.i)) { b.v = v; b.i = i; }
    }
    b = block_best(b, sm);
    if (b.i == 0x7fffffff) break;
    if (threadIdx.x == 0) { ov[r] = b.v; oi[r] = b.i; }
    pv = b.v; pi = b.i;
    got = r + 1;
  }
  return got;
}

__global__ void __launch_bounds__(256) topk_chunk_kernel(const float* __restrict__ logits, int V, int ld,
                                                          const float* __restrict__ temp, const int* __restrict__ top_k,
                                                          int idx_offset, Cand* __restrict__ cand, int n_chunks) {
  pdl_trigger();
  pdl_wait();
  __shared__ float cv[TOPK_CHUNK];
  __shared__ int ci[TOPK_CHUNK];
  __shared__ Best sm[32];
  __shared__ float ov[MAXK];
  __shared__ int oi[MAXK];
  const int n = blockIdx.x, c = blockIdx.y;
  const int K = clamp_k(top_k[n], temp[n]);
  const int lo = c * TOPK_CHUNK, cnt = min(TOPK_CHUNK, V - lo);
  const float* row = logits + (size_t)n * ld + lo;
  for (int j = threadIdx.x; j < cnt; j += blockDim.x) { cv[j] = row[j]; ci[j] = lo + j + idx_offset; }
  __syncthreads();
  const int got = select_topk(cv, ci, cnt, K, sm, ov, oi);
  __syncthreads();
  Cand* out = cand + ((size_t)n * n_chunks + c) * MAXK;
  for (int r = threadIdx.x; r < MAXK; r += blockDim.x)
    out[r] = r < got ? Cand{ov[r], oi[r]} : Cand{-INFINITY, 0x7fffffff};
}

// lists: [row][n_lists][MAXK] candidates. finish = 0: write the merged top-K to out_cand[row][MAXK] (padded with
// (-inf, INT_MAX)). finish = 1: nucleus + draw -> out_tok[row] and, when given, ids / probs / n_keep.
__global__ void __launch_bounds__(256) topk_merge_kernel(const Cand* __restrict__ lists, int n_lists, int list_row_stride,
                                                          const float* __restrict__ temp, const int* __restrict__ top_k,
                                                          const float* __restrict__ top_p, const float* __restrict__ u,
                                                          int finish, Cand* __restrict__ out_cand, int* __restrict__ out_tok,
                                                          int* __restrict__ ids, float* __restrict__ probs,
                                                          int* __restrict__ n_keep) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ unsigned char sraw[];
  __shared__ Best sm[32];
  __shared__ float ov[MAXK];
  __shared__ int oi[MAXK];
  const int n = blockIdx.x;
  const int total = n_lists * MAXK;
  float* cv = reinterpret_cast<float*>(sraw);
  int* ci = reinterpret_cast<int*>(sraw + (size_t)total * sizeof(float));
  const Cand* src = lists + (size_t)n * list_row_stride;
  for (int j = threadIdx.x; j < total; j += blockDim.x) { cv[j] = src[j].v; ci[j] = src[j].i; }
  __syncthreads();
  const float T = temp[n];
  const int K = clamp_k(top_k[n], T);
  const int got = select_topk(cv, ci, total, K, sm, ov, oi);
  __syncthreads();
  if (!finish) {
    for (int r = threadIdx.x; r < MAXK; r += blockDim.x)
      out_cand[(size_t)n * MAXK + r] = r < got ? Cand{ov[r], oi[r]} : Cand{-INFINITY, 0x7fffffff};
    return;
  }
  if (threadIdx.x == 0) {
    int keep = 1;
    int tok = got > 0 ? oi[0] : 0;
    if (T >= 1e-6f && got > 0) {
      const float mx = ov[0] / T;
      float sum = 0.f;
      for (int r = 0; r < got; ++r) { ov[r] = expf(ov[r] / T - mx); sum += ov[r]; }
      for (int r = 0; r < got; ++r) ov[r] /= sum;
      const float target = top_p[n];
      double cum = 0.0;
      keep = got;
      for (int r = 0; r < got; ++r) { cum += (double)ov[r]; if (cum >= (double)target) { keep = r + 1; break; } }
      double mass = 0.0;
      for (int r = 0; r < keep; ++r) mass += (double)ov[r];
      const double tgt = (double)(u ? u[n] : 0.f) * mass;
      double c = 0.0;
      tok = oi[keep - 1];
      for (int r = 0; r < keep; ++r) { c += (double)ov[r]; if (tgt < c) { tok = oi[r]; break; } }
    } else {
      ov[0] = 1.0f;
    }
    if (out_tok) out_tok[n] = tok;
    if (n_keep) n_keep[n] = keep;
    if (ids) for (int r = 0; r < keep; ++r) { ids[n * MAXK + r] = oi[r]; probs[n * MAXK + r] = ov[r]; }
  }
}

// One thread per lane. Columns [col0[l], col0[l] + nd[l]] are the lane's verify columns (nd drafts + 1); column t's
// nucleus scores draft t. result[l] = (accepted drafts, next token).
__global__ void spec_verify_kernel(const int* __restrict__ ids, const float* __restrict__ probs, const int* __restrict__ n_keep,
                                   const int* __restrict__ drafts, const float* __restrict__ u_acc,
                                   const float* __restrict__ u_ver, const int* __restrict__ col0, const int* __restrict__ nd,
                                   int n_lanes, int2* __restrict__ result) {
  pdl_trigger();
  pdl_wait();
  const int l = blockIdx.x * blockDim.x + threadIdx.x;
  if (l >= n_lanes) return;
  const int c0 = col0[l], D = nd[l];
  auto draw = [&](int col, int skip, double u) {
    const int* id = ids + (size_t)col * MAXK;
    const float* pr = probs + (size_t)col * MAXK;
    const int keep = n_keep[col];
    double mass = 0.0;
    int left = 0;
    for (int r = 0; r < keep; ++r) if (id[r] != skip) { mass += (double)pr[r]; ++left; }
    if (left == 0 || mass <= 0.0) {               // nothing left without the draft: the full nucleus
      skip = -1;
      mass = 0.0;
      for (int r = 0; r < keep; ++r) mass += (double)pr[r];
    }
    const double tgt = u * mass;
    double c = 0.0;
    int tok = -1, last = -1;
    for (int r = 0; r < keep; ++r) {
      if (id[r] == skip) continue;
      last = id[r];
      c += (double)pr[r];
      if (tgt < c) { tok = id[r]; break; }
    }
    return tok >= 0 ? tok : last;
  };
  for (int t = 0; t < D; ++t) {
    const int col = c0 + t, d = drafts[col];
    const int keep = n_keep[col];
    double mass = 0.0, pd = 0.0;
    for (int r = 0; r < keep; ++r) mass += (double)probs[(size_t)col * MAXK + r];
    for (int r = 0; r < keep; ++r) if (ids[(size_t)col * MAXK + r] == d) { pd = (double)probs[(size_t)col * MAXK + r] / mass; break; }
    if ((double)u_acc[col] < pd) continue;
    result[l] = make_int2(t, draw(col, d, (double)u_ver[col]));
    return;
  }
  result[l] = make_int2(D, draw(c0 + D, -1, (double)u_ver[c0 + D]));
}

}  // namespace

extern "C" int vg_argmax(const float* logits, int N, int V, int ld, int* out, float* out_val, int idx_offset,
                         cudaStream_t st) {
  if (N <= 0) return 0;
  launch_pdl(argmax_kernel, dim3(N), dim3(1024), 0, st, logits, V, ld, out, out_val, idx_offset);
  return (int)cudaGetLastError();
}

extern "C" int vg_penalty(float* logits, int N, int V, int ld, const int* toks, const int* counts, const int* n_toks,
                          int max_toks, const float* rep, const float* pres, const float* freq, int idx_offset,
                          cudaStream_t st) {
  if (N <= 0) return 0;
  return (int)launch_pdl(penalty_kernel, dim3(N), dim3(64), 0, st, logits, ld, toks, counts, n_toks, max_toks, rep, pres, freq,
                         V, idx_offset);
}

extern "C" int vg_topk_chunks(int V) { return (V + TOPK_CHUNK - 1) / TOPK_CHUNK; }

// Local top-K of every row: chunk pass + merge. cand_chunks: scratch of N * vg_topk_chunks(V) * 64 pairs; out_cand:
// N * 64 (value, index + idx_offset) pairs in selection order, padded with (-inf, INT_MAX).
extern "C" int vg_topk_local(const float* logits, int N, int V, int ld, const float* temp, const int* top_k, int idx_offset,
                             void* cand_chunks, void* out_cand, cudaStream_t st) {
  if (N <= 0) return 0;
  const int C = vg_topk_chunks(V);
  if (C * MAXK * 8 > 200 * 1024) return -2;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(topk_merge_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  cudaError_t e = launch_pdl(topk_chunk_kernel, dim3(N, C), dim3(256), 0, st, logits, V, ld, temp, top_k, idx_offset,
                             static_cast<Cand*>(cand_chunks), C);
  if (e != cudaSuccess) return (int)e;
  return (int)launch_pdl(topk_merge_kernel, dim3(N), dim3(256), (size_t)C * MAXK * 8, st, static_cast<const Cand*>(cand_chunks), C,
                         C * MAXK, temp, top_k, (const float*)nullptr, (const float*)nullptr, 0, static_cast<Cand*>(out_cand),
                         (int*)nullptr, (int*)nullptr, (float*)nullptr, (int*)nullptr);
}

// Nucleus + draw from `n_lists` top-K lists per row (lists[row * row_stride_pairs + list * 64 + r]): one list on a single
// GPU, one per rank after the all-gather of the ranks' local lists. u[row] in [0, 1) drives the draw.
extern "C" int vg_nucleus_finish(const void* lists, int n_lists, int row_stride_pairs, int N, const float* temp, const int* top_k,
                                 const float* top_p, const float* u, int* out_tok, int* ids, float* probs, int* n_keep,
                                 cudaStream_t st) {
  if (N <= 0) return 0;
  if (n_lists < 1 || n_lists > 64) return -2;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(topk_merge_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return (int)launch_pdl(topk_merge_kernel, dim3(N), dim3(256), (size_t)n_lists * MAXK * 8, st, static_cast<const Cand*>(lists),
                         n_lists, row_stride_pairs, temp, top_k, top_p, u, 1, (Cand*)nullptr, out_tok, ids, probs, n_keep);
}

extern "C" int vg_spec_verify(const int* ids, const float* probs, const int* n_keep, const int* drafts, const float* u_acc,
                              const float* u_ver, const int* col0, const int* nd, int n_lanes, int* result, cudaStream_t st) {
  if (n_lanes <= 0) return 0;
  return (int)launch_pdl(spec_verify_kernel, dim3((n_lanes + 31) / 32), dim3(32), 0, st, ids, probs, n_keep, drafts, u_acc, u_ver,
                         col0, nd, n_lanes, reinterpret_cast<int2*>(result));
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

// Peer-memory collectives over NVLink / NVSwitch for tensor and expert parallelism (one process per GPU).
//
// Substrate: every rank cudaMalloc's one "symmetric" arena of the same size, exports it with a CUDA IPC
// handle and maps every peer's arena; kernels then use plain ld/st on the peer pointers. The arena holds
//   flags   [4 sets][8 source ranks][64 CTAs] one 32-bit flag per 128-byte line (sets 2,3: second phase)
//   slots   [2 sets][8 source ranks][slot_bytes] receive buffers, written by the source rank
//   result  [2 sets][result_bytes] all-gather landing zone of the two-shot all-reduce
// plus a device-resident epoch counter, so a kernel captured in a CUDA graph advances its own epoch on
// every replay. Epoch e uses set e & 1: a rank can only start epoch e+2 after it has seen every peer's
// epoch e+1 flag, which the peer sets after it finished reading epoch e, so two sets are enough.
//
// All reductions add the ranks' fp32 partials in rank order 0..W-1 on every rank: results are bit-identical
// across ranks and run to run. Waits on peer flags are bounded by a wall-clock budget; on expiry the kernel
// stores an error code in the status word and returns (no trap, no hang), the device-side analogue of the
// reference's cooperative abort word (reference: native/tp_doorbell.h:24-31, kernels/gpu_batch.cu:141-238,
// native/net_shim.c:457-623 describe the two-box doorbell transport this replaces).
//
// No multimem / NVLS and no TMA multicast are used here: only plain peer loads and stores.
#include "common.cuh"
#include "api.h"

namespace {
using namespace vg;

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// Rank-order sum of eight consecutive fp32 elements over the W receive slots (16-byte loads through L2).
__device__ __forceinline__ void sum8_ranks(const float* base, size_t stride, size_t i, int W, float* s) {
#pragma unroll
  for (int k = 0; k < 8; ++k) s[k] = 0.f;
  for (int q = 0; q < W; ++q) {
    const float4 a = __ldcg(reinterpret_cast<const float4*>(base + (size_t)q * stride + i));
    const float4 b = __ldcg(reinterpret_cast<const float4*>(base + (size_t)q * stride + i) + 1);
    s[0] += a.x; s[1] += a.y; s[2] += a.z; s[3] += a.w;
    s[4] += b.x; s[5] += b.y; s[6] += b.z; s[7] += b.w;
  }
}
__device__ __forceinline__ uint4 pack_bf16x8(const float* s) {
  uint4 o;
  __nv_bfloat16* b = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
  for (int k = 0; k < 8; ++k) b[k] = __float2bfloat16_rn(s[k]);
  return o;
}
template <typename T> __device__ __forceinline__ void load8_f32(const T* p, float* v);
template <> __device__ __forceinline__ void load8_f32<float>(const float* p, float* v) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *(reinterpret_cast<const float4*>(p) + 1);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <> __device__ __forceinline__ void load8_f32<__nv_bfloat16>(const __nv_bfloat16* p, float* v) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(&u);
#pragma unroll
  for (int k = 0; k < 8; ++k) v[k] = __bfloat162float(b[k]);
}

// One-shot all-reduce: every rank pushes its whole vector (as fp32) into its slot on every rank, raises a
// per-CTA flag there, waits for the W flags of its own chunk and sums the W slots in rank order.
template <typename TIn>
__global__ void __launch_bounds__(256) allreduce_oneshot_kernel(VgCommCtx c, const TIn* __restrict__ in,
                                                                 __nv_bfloat16* __restrict__ out_bf, float* __restrict__ out_f32,
                                                                 int n) {
  __shared__ int failed;
  const uint32_t e = *c.epoch + 1;
  const int set = e & 1;
  const int cta = blockIdx.x, nct = gridDim.x;
  const int per = ((n + nct - 1) / nct + 3) & ~3;
  const int lo = min(n, cta * per), hi = min(n, lo + per);
  if (threadIdx.x == 0) failed = 0;
  for (int p = 0; p < c.world; ++p) {
    const int peer = (c.rank + p) % c.world;          // start with a different peer on every rank
    float* dst = reinterpret_cast<float*>(c.data[peer] + c.slots_off + (size_t)(set * MAX_RANKS + c.rank) * c.slot_bytes);
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) dst[i] = to_f32<TIn>(in[i]);
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < c.world) {
    uint32_t* f = reinterpret_cast<uint32_t*>(c.data[threadIdx.x] + c.flags_off) + flag_index(set, c.rank, cta);
    st_release_sys(f, e);
  }
  if (threadIdx.x < c.world) {
    const uint32_t* f = reinterpret_cast<const uint32_t*>(c.data[c.rank] + c.flags_off) + flag_index(set, threadIdx.x, cta);
    if (!wait_flag(f, e, c.timeout_ns)) { atomicCAS(c.status, 0, VG_ERR_PEER_WAIT); failed = 1; }
  }
  __syncthreads();
  if (!failed) {
    const float* base = reinterpret_cast<const float*>(c.data[c.rank] + c.slots_off + (size_t)set * MAX_RANKS * c.slot_bytes);
    const size_t stride = c.slot_bytes / sizeof(float);
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
      float s = 0.f;
      for (int q = 0; q < c.world; ++q) s += __ldcg(&base[(size_t)q * stride + i]);
      if (out_bf) out_bf[i] = __float2bfloat16_rn(s);
      if (out_f32) out_f32[i] = s;
    }
  }
  // the last CTA to finish publishes the new epoch for the next launch
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(c.done_ctr, 1u) == (unsigned)nct - 1) { *c.done_ctr = 0; *c.epoch = e; }
  }
}

// Two-shot all-reduce for long vectors: reduce-scatter (rank r owns segment r and receives every rank's
// partial of it), rank-order sum, then all-gather by pushing the reduced bf16 segment into every rank's
// result area. Each CTA handles the same sub-chunk of every segment and uses its own flags.
template <typename TIn>
__global__ void __launch_bounds__(256) allreduce_twoshot_kernel(VgCommCtx c, const TIn* __restrict__ in,
                                                                 __nv_bfloat16* __restrict__ out, int n) {
  __shared__ int failed;
  const uint32_t e = *c.epoch + 1;
  const int set = e & 1;
  const int W = c.world, cta = blockIdx.x, nct = gridDim.x;
  const int seg = ((n + W - 1) / W + 7) & ~7;                    // elements per segment
  const int per = ((seg + nct - 1) / nct + 7) & ~7;              // elements per CTA within a segment
  const int lo = min(seg, cta * per), hi = min(seg, lo + per);
  const bool vec = (n & 7) == 0 && ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  if (threadIdx.x == 0) failed = 0;
  // phase 1: push my partial of segment p to rank p
  for (int k = 0; k < W; ++k) {
    const int p = (c.rank + k) % W;
    float* dst = reinterpret_cast<float*>(c.data[p] + c.slots_off + (size_t)(set * MAX_RANKS + c.rank) * c.slot_bytes);
    const int g0 = p * seg;
    if (vec) {
      // eight elements per thread, 16-byte stores over NVLink (n, seg, lo, hi are multiples of 8)
      for (int i = lo + 8 * (int)threadIdx.x; i < hi; i += 8 * (int)blockDim.x) {
        const int g = g0 + i;
        float v[8];
        if (g < n) {
          load8_f32<TIn>(in + g, v);
        } else {
#pragma unroll
          for (int k = 0; k < 8; ++k) v[k] = 0.f;
        }
        reinterpret_cast<float4*>(dst + i)[0] = make_float4(v[0], v[1], v[2], v[3]);
        reinterpret_cast<float4*>(dst + i)[1] = make_float4(v[4], v[5], v[6], v[7]);
      }
    } else {
      for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const int g = g0 + i;
        dst[i] = g < n ? to_f32<TIn>(in[g]) : 0.f;
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < W)
    st_release_sys(reinterpret_cast<uint32_t*>(c.data[threadIdx.x] + c.flags_off) + flag_index(set, c.rank, cta), e);
  if (threadIdx.x < W) {
    const uint32_t* f = reinterpret_cast<const uint32_t*>(c.data[c.rank] + c.flags_off) + flag_index(set, threadIdx.x, cta);
    if (!wait_flag(f, e, c.timeout_ns)) { atomicCAS(c.status, 0, VG_ERR_PEER_WAIT); failed = 1; }
  }
  __syncthreads();
  // phase 2: reduce my segment in rank order and push it to everyone's result area
  if (!failed) {
    const float* base = reinterpret_cast<const float*>(c.data[c.rank] + c.slots_off + (size_t)set * MAX_RANKS * c.slot_bytes);
    const size_t stride = c.slot_bytes / sizeof(float);
    // (lo, hi and seg are multiples of 8: eight elements per thread, one 16-byte store per peer)
    for (int i = lo + 8 * (int)threadIdx.x; i < hi; i += 8 * (int)blockDim.x) {
      float s[8];
      sum8_ranks(base, stride, (size_t)i, W, s);
      const uint4 v = pack_bf16x8(s);
      const size_t g = (size_t)c.rank * seg + i;
      for (int k = 0; k < W; ++k) {
        const int p = (c.rank + k) % W;
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(c.data[p] + c.result_off + (size_t)set * c.result_bytes) + g) = v;
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  // second flag round: set index 2 + set keeps it apart from phase 1
  if (threadIdx.x < W)
    st_release_sys(reinterpret_cast<uint32_t*>(c.data[threadIdx.x] + c.flags_off) + flag_index(2 + set, c.rank, cta), e);
  if (threadIdx.x < W) {
    const uint32_t* f = reinterpret_cast<const uint32_t*>(c.data[c.rank] + c.flags_off) + flag_index(2 + set, threadIdx.x, cta);
    if (!wait_flag(f, e, c.timeout_ns)) { atomicCAS(c.status, 0, VG_ERR_PEER_WAIT); failed = 1; }
  }
  __syncthreads();
  if (!failed) {
    const __nv_bfloat16* res = reinterpret_cast<const __nv_bfloat16*>(c.data[c.rank] + c.result_off + (size_t)set * c.result_bytes);
    for (int q = 0; q < W; ++q) {
      if (vec) {
        for (int i = lo + 8 * (int)threadIdx.x; i < hi; i += 8 * (int)blockDim.x) {
          const size_t g = (size_t)q * seg + i;
          if (g < (size_t)n) *reinterpret_cast<uint4*>(out + g) = __ldcg(reinterpret_cast<const uint4*>(res + g));
        }
      } else {
        for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
          const size_t g = (size_t)q * seg + i;
          if (g < (size_t)n) out[g] = __ldcg(&res[g]);
        }
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(c.done_ctr, 1u) == (unsigned)nct - 1) { *c.done_ctr = 0; *c.epoch = e; }
  }
}

// In-switch all-reduce of a bf16 buffer that lives in multicast-bound symmetric memory (same offset on every rank),
// in place: after a flag round (every rank's producer has finished writing its copy), rank r reads the sum of all
// ranks' copies of slice r with multimem.ld_reduce (fp32 accumulation inside the NVLink switch) and writes it to every
// rank's copy with multimem.st; a second flag round makes the result complete everywhere. Every element crosses each
// GPU's links once in and once out, and every rank ends with identical bits.
__global__ void __launch_bounds__(256) allreduce_multimem_kernel(VgCommCtx c, unsigned char* mc_buf, long long n8) {
  __shared__ int failed;
  const uint32_t e = *c.epoch + 1;
  const int set = e & 1;
  const int W = c.world, cta = blockIdx.x, nct = gridDim.x;
  if (threadIdx.x == 0) failed = 0;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < W)
    st_release_sys(reinterpret_cast<uint32_t*>(c.data[threadIdx.x] + c.flags_off) + flag_index(set, c.rank, cta), e);
  if (threadIdx.x < W) {
    const uint32_t* f = reinterpret_cast<const uint32_t*>(c.data[c.rank] + c.flags_off) + flag_index(set, threadIdx.x, cta);
    if (!wait_flag(f, e, c.timeout_ns)) { atomicCAS(c.status, 0, VG_ERR_PEER_WAIT); failed = 1; }
  }
  __syncthreads();
  if (!failed) {
    const long long seg = (n8 + W - 1) / W;                       // 16-byte vectors per rank
    const long long lo = c.rank * seg, hi = min(n8, lo + seg);
    for (long long i = lo + (long long)cta * blockDim.x + threadIdx.x; i < hi; i += (long long)nct * blockDim.x) {
      const uint4 v = multimem_ld_reduce_bf16x8(mc_buf + i * 16);
      multimem_st_bf16x8(mc_buf + i * 16, v);
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < W)
    st_release_sys(reinterpret_cast<uint32_t*>(c.data[threadIdx.x] + c.flags_off) + flag_index(2 + set, c.rank, cta), e);
  if (threadIdx.x < W) {
    const uint32_t* f = reinterpret_cast<const uint32_t*>(c.data[c.rank] + c.flags_off) + flag_index(2 + set, threadIdx.x, cta);
    if (!wait_flag(f, e, c.timeout_ns)) { atomicCAS(c.status, 0, VG_ERR_PEER_WAIT); failed = 1; }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(c.done_ctr, 1u) == (unsigned)nct - 1) { *c.done_ctr = 0; *c.epoch = e; }
  }
}

// All-gather of a small payload (<= slot_bytes) from every rank: out[q * bytes ...] = rank q's payload.
// ------------------------------------------------------------------ fused all-gather + GEMM: the gather half
// grid (tiles of 128 rows, column chunks). Each CTA copies its chunk of its tile into every rank's landing zone;
// the last CTA of a tile (local counter) publishes the tile's epoch word on every rank.
__global__ void __launch_bounds__(256) ag_push_kernel(VgCommCtx c, const __half* __restrict__ x, int row0, int rows, int K,
                                                      unsigned int* __restrict__ tile_ctr) {
  __shared__ int last;
  const uint32_t e = *c.epoch + 1;
  const int set = e & 1;
  const int t = blockIdx.x, chunks = gridDim.y, ch = blockIdx.y;
  const int r_lo = t * 128, r_hi = min(rows, r_lo + 128);
  const int vec_per_row = K / 8;                                    // 16-byte vectors per row
  const int v_lo = (int)((long long)vec_per_row * ch / chunks), v_hi = (int)((long long)vec_per_row * (ch + 1) / chunks);
  const int vw = v_hi - v_lo;
  // two landing zones, picked by the epoch's parity: a fast rank may push the next gather while a slow one still reads
  const size_t cap_rows = (size_t)(c.agbuf_bytes / 2 / ((unsigned long long)K * 2ull)) / 128 * 128;
  for (int k = 0; k < c.world; ++k) {
    const int p = (c.rank + k) % c.world;
    __half* dst = reinterpret_cast<__half*>(c.data[p] + c.agbuf_off) + (size_t)set * cap_rows * K;
    for (int i = threadIdx.x; i < (r_hi - r_lo) * vw; i += blockDim.x) {
      const int r = r_lo + i / vw, v = v_lo + i % vw;
      const uint4 val = *reinterpret_cast<const uint4*>(x + (size_t)r * K + v * 8);
      *reinterpret_cast<uint4*>(dst + (size_t)(row0 + r) * K + v * 8) = val;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) last = atomicAdd(&tile_ctr[t], 1u) == (unsigned)chunks - 1;
  __syncthreads();
  if (last) {
    if (threadIdx.x == 0) tile_ctr[t] = 0;
    __threadfence_system();
    if (threadIdx.x < c.world)
      st_release_sys(reinterpret_cast<uint32_t*>(c.data[threadIdx.x] + c.agflags_off) + (size_t)set * VG_AG_MAX_TILES +
                         (row0 / 128 + t), e);
  }
}

// ------------------------------------------------------------------ fused GEMM + reduce-scatter: second half
// Every rank's row-parallel GEMM pushed its fp32 partial tiles of this rank's token rows into this rank's slots and
// published one epoch word per tile (csrc/gemm_tc.cu, rs epilogue). Here: wait for the tiles of every rank,
// sum in rank order, push the bf16 result into every rank's result area, wait for the other segments, assemble
// `out`. Same second flag round, completion counter and epoch update as the two-shot all-reduce.
__global__ void __launch_bounds__(256) gemm_rs_finish_kernel(VgCommCtx c, __nv_bfloat16* __restrict__ out, int n, int M,
                                                             int rs_rows, int m_tiles) {
  __shared__ int failed;
  const uint32_t e = *c.epoch + 1;
  const int set = e & 1;
  const int W = c.world, cta = blockIdx.x, nct = gridDim.x;
  const int my0 = c.rank * rs_rows, my_rows = max(0, min(n, my0 + rs_rows) - my0);
  const int my_tiles = ((my_rows + 127) / 128) * m_tiles;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  // every tile of my rows from every rank
  {
    const uint32_t* fl = reinterpret_cast<const uint32_t*>(c.data[c.rank] + c.rsflags_off);
    for (int i = threadIdx.x; i < W * my_tiles; i += blockDim.x) {
      const int q = i / my_tiles, t = i % my_tiles;
      if (!wait_flag(fl + ((size_t)(set * MAX_RANKS + q) * VG_RS_MAX_TILES + t), e, c.timeout_ns)) {
        atomicCAS(c.status, 0, VG_ERR_PEER_WAIT);
        failed = 1;
      }
    }
  }
  __syncthreads();
  const size_t seg = (size_t)rs_rows * M;                          // elements per owner segment
  const size_t mine = (size_t)my_rows * M;
  const size_t per = ((mine + nct - 1) / nct + 7) & ~(size_t)7;
  const size_t lo = min(mine, (size_t)cta * per), hi = min(mine, lo + per);
  if (!failed) {
    const float* base = reinterpret_cast<const float*>(c.data[c.rank] + c.slots_off + (size_t)set * MAX_RANKS * c.slot_bytes);
    const size_t stride = c.slot_bytes / sizeof(float);
    // (M is a multiple of 8, so are lo, hi and seg: eight elements per thread, one 16-byte store per peer)
    for (size_t i = lo + 8 * (size_t)threadIdx.x; i < hi; i += 8 * (size_t)blockDim.x) {
      float s[8];
      sum8_ranks(base, stride, i, W, s);
      const uint4 v = pack_bf16x8(s);
      const size_t g = (size_t)c.rank * seg + i;
      for (int k = 0; k < W; ++k) {
        const int p = (c.rank + k) % W;
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(c.data[p] + c.result_off + (size_t)set * c.result_bytes) + g) = v;
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < W)
    st_release_sys(reinterpret_cast<uint32_t*>(c.data[threadIdx.x] + c.flags_off) + flag_index(2 + set, c.rank, cta), e);
  if (threadIdx.x < W) {
    const uint32_t* f = reinterpret_cast<const uint32_t*>(c.data[c.rank] + c.flags_off) + flag_index(2 + set, threadIdx.x, cta);
    if (!wait_flag(f, e, c.timeout_ns)) { atomicCAS(c.status, 0, VG_ERR_PEER_WAIT); failed = 1; }
  }
  __syncthreads();
  if (!failed) {
    // CTA `cta` of every rank covered the same relative slice of its own segment: copy those slices
    const __nv_bfloat16* res = reinterpret_cast<const __nv_bfloat16*>(c.data[c.rank] + c.result_off + (size_t)set * c.result_bytes);
    const size_t total = (size_t)n * M;
    for (int q = 0; q < W; ++q) {
      const int q_rows = max(0, min(n, (q + 1) * rs_rows) - q * rs_rows);
      const size_t qn = (size_t)q_rows * M;
      const size_t qper = ((qn + nct - 1) / nct + 7) & ~(size_t)7;
      const size_t qlo = min(qn, (size_t)cta * qper), qhi = min(qn, qlo + qper);
      for (size_t i = qlo + 8 * (size_t)threadIdx.x; i < qhi; i += 8 * (size_t)blockDim.x) {
        const size_t g = (size_t)q * seg + i;
        if (g < total) *reinterpret_cast<uint4*>(out + g) = __ldcg(reinterpret_cast<const uint4*>(res + g));
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(c.done_ctr, 1u) == (unsigned)nct - 1) { *c.done_ctr = 0; *c.epoch = e; }
  }
}

__global__ void __launch_bounds__(256) allgather_small_kernel(VgCommCtx c, const uint8_t* __restrict__ in,
                                                               uint8_t* __restrict__ out, int bytes) {
  __shared__ int failed;
  const uint32_t e = *c.epoch + 1;
  const int set = e & 1;
  if (threadIdx.x == 0) failed = 0;
  for (int p = 0; p < c.world; ++p) {
    uint8_t* dst = c.data[p] + c.slots_off + (size_t)(set * MAX_RANKS + c.rank) * c.slot_bytes;
    for (int i = threadIdx.x; i < bytes; i += blockDim.x) dst[i] = in[i];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < c.world)
    st_release_sys(reinterpret_cast<uint32_t*>(c.data[threadIdx.x] + c.flags_off) + flag_index(set, c.rank, 0), e);
  if (threadIdx.x < c.world) {
    const uint32_t* f = reinterpret_cast<const uint32_t*>(c.data[c.rank] + c.flags_off) + flag_index(set, threadIdx.x, 0);
    if (!wait_flag(f, e, c.timeout_ns)) { atomicCAS(c.status, 0, VG_ERR_PEER_WAIT); failed = 1; }
  }
  __syncthreads();
  if (!failed) {
    for (int q = 0; q < c.world; ++q) {
      const uint8_t* src = c.data[c.rank] + c.slots_off + (size_t)(set * MAX_RANKS + q) * c.slot_bytes;
      for (int i = threadIdx.x; i < bytes; i += blockDim.x) out[(size_t)q * bytes + i] = __ldcg(&src[i]);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) { __threadfence(); *c.epoch = e; }
}

// Vocabulary-parallel arg-max merge: pairs[q][col] = (value, global index) from rank q; the winner is the
// largest value, lowest index on ties (rank order == ascending vocabulary order).
__global__ void argmax_merge_kernel(const float* __restrict__ pairs, int world, int ncols, int* __restrict__ out) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= ncols) return;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int q = 0; q < world; ++q) {
    const float v = pairs[((size_t)q * ncols + col) * 2];
    const int i = __float_as_int(pairs[((size_t)q * ncols + col) * 2 + 1]);
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
  }
  out[col] = bi;
}

__global__ void pack_pairs_kernel(const float* __restrict__ val, const int* __restrict__ idx, int n, float* __restrict__ out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) { out[2 * i] = val[i]; out[2 * i + 1] = __int_as_float(idx[i]); }
}

// A wait that nothing satisfies: exercises the bounded-wait error path without any peer (tests only use
// it with a short budget; the context stays usable).
__global__ void wait_timeout_probe_kernel(VgCommCtx c, unsigned long long budget_ns) {
  const uint32_t* f = reinterpret_cast<const uint32_t*>(c.data[c.rank] + c.flags_off) + flag_index(3, MAX_RANKS - 1, MAX_CTAS - 1);
  if (!wait_flag(f, 0x7fffffffu, budget_ns)) atomicCAS(c.status, 0, VG_ERR_PEER_WAIT);
}

}  // namespace

// ------------------------------------------------------------------ host API

extern "C" int vg_comm_alloc(void** ptr, unsigned long long bytes) {
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemset(*ptr, 0, bytes);
}
extern "C" int vg_comm_free(void* ptr) { return (int)cudaFree(ptr); }
extern "C" int vg_comm_export(void* ptr, void* handle64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) return (int)e;
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
extern "C" int vg_comm_import(const void* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  return (int)cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
}
extern "C" int vg_comm_close(void* ptr) { return (int)cudaIpcCloseMemHandle(ptr); }
extern "C" int vg_comm_handle_bytes(void) { return (int)sizeof(cudaIpcMemHandle_t); }

static int pick_ctas(long long n, int max_ctas) {
  long long c = (n + 4095) / 4096;
  if (c < 1) c = 1;
  if (c > max_ctas) c = max_ctas;
  return (int)c;
}

extern "C" int vg_comm_allreduce(const VgCommCtx* ctx, const void* in, int in_is_f32, void* out_bf16, float* out_f32,
                                 long long n, cudaStream_t st) {
  if (n <= 0) return 0;
  const VgCommCtx c = *ctx;
  if (c.world < 1 || c.world > MAX_RANKS) return -2;
  const bool one_shot = (unsigned long long)n * 4ull <= c.slot_bytes && n <= (1 << 20);
  if (one_shot) {
    const int ctas = pick_ctas(n, 32);
    if (in_is_f32)
      allreduce_oneshot_kernel<float><<<ctas, 256, 0, st>>>(c, static_cast<const float*>(in), static_cast<__nv_bfloat16*>(out_bf16), out_f32, (int)n);
    else
      allreduce_oneshot_kernel<__nv_bfloat16><<<ctas, 256, 0, st>>>(c, static_cast<const __nv_bfloat16*>(in), static_cast<__nv_bfloat16*>(out_bf16), out_f32, (int)n);
    return (int)cudaGetLastError();
  }
  const long long seg = (((n + c.world - 1) / c.world) + 7) & ~7ll;
  if ((unsigned long long)seg * 4ull > c.slot_bytes || (unsigned long long)seg * c.world * 2ull > c.result_bytes || out_f32) return -3;
  const int ctas = pick_ctas(seg, MAX_CTAS);
  if (in_is_f32)
    allreduce_twoshot_kernel<float><<<ctas, 256, 0, st>>>(c, static_cast<const float*>(in), static_cast<__nv_bfloat16*>(out_bf16), (int)n);
  else
    allreduce_twoshot_kernel<__nv_bfloat16><<<ctas, 256, 0, st>>>(c, static_cast<const __nv_bfloat16*>(in), static_cast<__nv_bfloat16*>(out_bf16), (int)n);
  return (int)cudaGetLastError();
}

// In-place in-switch all-reduce of `n` bf16 elements at the multicast address `mc_buf` (n a multiple of 8, buffer
// 16-byte aligned and bound to the same multicast object on every rank).
extern "C" int vg_comm_allreduce_multimem(const VgCommCtx* ctx, void* mc_buf, long long n, cudaStream_t st) {
  if (n <= 0) return 0;
  if (!ctx || ctx->world < 2 || !mc_buf || (n % 8) != 0 || (reinterpret_cast<uintptr_t>(mc_buf) & 15) != 0) return -2;
  allreduce_multimem_kernel<<<MAX_CTAS, 256, 0, st>>>(*ctx, static_cast<unsigned char*>(mc_buf), n / 8);
  return (int)cudaGetLastError();
}

namespace { unsigned int* g_ag_ctr[64] = {}; }
extern "C" int vg_comm_ag_push(const VgCommCtx* ctx, const void* x_f16, int row0, int rows, int K, cudaStream_t st) {
  if (!ctx || ctx->world < 2 || rows < 0 || (row0 % 128) != 0 || (K % 8) != 0) return -2;
  const long long cap_rows = (long long)(ctx->agbuf_bytes / 2 / ((unsigned long long)K * 2ull)) / 128 * 128;
  if ((row0 + rows + 127) / 128 > VG_AG_MAX_TILES || row0 + rows > cap_rows) return -5;
  if (rows == 0) return 0;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return -2;
  if (!g_ag_ctr[dev]) {                                   // per-tile arrival counters, allocated once per device
    cudaError_t e = cudaMalloc(&g_ag_ctr[dev], VG_AG_MAX_TILES * sizeof(unsigned int));
    if (e != cudaSuccess) return (int)e;
    e = cudaMemset(g_ag_ctr[dev], 0, VG_AG_MAX_TILES * sizeof(unsigned int));
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid((rows + 127) / 128, 8);
  ag_push_kernel<<<grid, 256, 0, st>>>(*ctx, static_cast<const __half*>(x_f16), row0, rows, K, g_ag_ctr[dev]);
  return (int)cudaGetLastError();
}

extern "C" int vg_comm_gemm_rs_finish(const VgCommCtx* ctx, void* out_bf16, int n, int M, int rs_rows, cudaStream_t st) {
  if (!ctx || ctx->world < 2 || n <= 0 || M <= 0 || rs_rows <= 0 || (rs_rows % 128) != 0) return -2;
  if ((M % 8) != 0 || (reinterpret_cast<uintptr_t>(out_bf16) & 15) != 0) return -2;      // 16-byte accesses throughout
  const int m_tiles = (M + 127) / 128;
  if ((long long)(rs_rows / 128) * m_tiles > VG_RS_MAX_TILES || (unsigned long long)rs_rows * M * 4ull > ctx->slot_bytes ||
      (unsigned long long)rs_rows * ctx->world * M * 2ull > ctx->result_bytes)
    return -5;
  int ctas = (int)(((long long)rs_rows * M + 256 * 32 - 1) / (256 * 32));
  ctas = ctas < 1 ? 1 : (ctas > MAX_CTAS ? MAX_CTAS : ctas);
  gemm_rs_finish_kernel<<<ctas, 256, 0, st>>>(*ctx, static_cast<__nv_bfloat16*>(out_bf16), n, M, rs_rows, m_tiles);
  return (int)cudaGetLastError();
}

extern "C" int vg_comm_allgather_small(const VgCommCtx* ctx, const void* in, void* out, int bytes, cudaStream_t st) {
  const VgCommCtx c = *ctx;
  if (bytes <= 0 || (unsigned long long)bytes > c.slot_bytes) return -2;
  allgather_small_kernel<<<1, 256, 0, st>>>(c, static_cast<const uint8_t*>(in), static_cast<uint8_t*>(out), bytes);
  return (int)cudaGetLastError();
}

// Local arg-max values/indices (already offset to global vocabulary ids) -> global arg-max on every rank.
extern "C" int vg_comm_argmax_merge(const VgCommCtx* ctx, const float* val, const int* idx, int ncols, float* scratch_pairs,
                                    float* gathered, int* out, cudaStream_t st) {
  const VgCommCtx c = *ctx;
  if (ncols < 1 || ncols > VG_ARGMAX_MAX_COLS) return -2;      // the wrappers' pair / gather buffers hold this many columns
  pack_pairs_kernel<<<(ncols + 127) / 128, 128, 0, st>>>(val, idx, ncols, scratch_pairs);
  int rc = vg_comm_allgather_small(ctx, scratch_pairs, gathered, ncols * 8, st);
  if (rc) return rc;
  argmax_merge_kernel<<<(ncols + 127) / 128, 128, 0, st>>>(gathered, c.world, ncols, out);
  return (int)cudaGetLastError();
}

extern "C" int vg_comm_wait_timeout_probe(const VgCommCtx* ctx, unsigned long long budget_ns, cudaStream_t st) {
  wait_timeout_probe_kernel<<<1, 1, 0, st>>>(*ctx, budget_ns);
  return (int)cudaGetLastError();
}

// GatedDeltaNet prefill in chunked (WY / UT-transform) form on the tensor cores (tcgen05.mma kind::tf32, fp32
// accumulators in TMEM). The recurrence of one value head with state S [kd, vd],
//     S_t = g_t S_{t-1} + k_t d_t^T,   d_t = beta_t (v_t - (g_t S_{t-1})^T k_t),   o_t = S_t^T q_t,
// is evaluated 64 tokens at a time. With G_i = sum_{j<=i} log g_j inside a chunk, A_ij = beta_i e^{G_i-G_j} (k_i.k_j)
// for j < i and T = (I + A)^-1 (unit lower triangular):
//     W = T diag(beta e^G) K          U = T diag(beta) V          D = U - W S_0            (the chunk's deltas)
//     O = diag(e^G) Q S_0 + (M o Q K^T) D,   M_ij = e^{G_i-G_j} [j <= i]
//     S_C = e^{G_C} S_0 + (diag(e^{G_C-G}) K)^T D
// Everything that does not involve S_0 is independent per chunk and runs first, for all chunks at once
// (gdn_chunk_prep_kernel: grid = value heads x pairs of chunks); the part that carries the state runs as one CTA per
// value head walking its chunks (gdn_chunk_scan_kernel), four small GEMMs per chunk. The reference evaluates the
// same recurrence token by token on CUDA cores (reference: kernels/gpu_batch.cu:580 delta_step_prefill, :439-444);
// the chunked form exists only for prefill. Decode and verify keep the exact step kernel, so the batch-invariance
// contract (verify == sequential decode, bit for bit) is untouched; a prefill through this path agrees with the
// step kernel to tf32 rounding (~1e-3 relative), not bit for bit.
//
// All operand tiles handed from the first kernel to the second are stored in global memory as ready-made images of
// the shared-memory layout the MMA reads (K-major, 128-byte swizzle, 32-bit elements), so the second kernel's loads
// are plain bulk copies. Every wait is bounded.
#include "common.cuh"
#include "api.h"

namespace {
using namespace vg;

constexpr int CH = 64;                    // chunk length
constexpr int KD = 128, VD = 128;
// Per (head, chunk) record in global memory. Operands that share an A operand in the state-carrying kernel are stacked
// into ONE image, so one MMA sequence serves both (a kind::tf32 MMA covers only K = 8 and small MMAs retire at about
// one per 100 cycles: the instruction count, not the FLOPs, is what the serial chain pays for):
//   WQ   [128 rows][128 k]  rows 0..63 = W (row i), rows 64..127 = e^G Q (row i)
//   PK   [192 rows][64 j]   rows 0..63 = P (row i), rows 64..191 = K~^T (row d)
//   UT   plain fp32 [128 v][64 i]
constexpr uint32_t WQ_IMG = 2 * CH * KD * 4;        // 64 KB
constexpr uint32_t PK_IMG = (CH + KD) * CH * 4;     // 48 KB
constexpr uint32_t UT_BYTES = VD * CH * 4;          // 32 KB
constexpr uint32_t CHUNK_BYTES = WQ_IMG + PK_IMG + UT_BYTES;   // 144 KB per (head, chunk)

// Byte offset of element (r, k) in the image of a K-major tile of `rows` rows of 32-bit elements with the 128-byte
// swizzle: 32 elements (128 bytes) of a row are contiguous, the 16-byte pieces of a row are XOR-ed with r & 7, and
// successive groups of 32 k-values are whole [rows x 128 B] panels.
__host__ __device__ __forceinline__ uint32_t img_off(int rows, int r, int k) {
  const int panel = k >> 5, kk = k & 31;
  return (uint32_t)(panel * rows * 128 + r * 128 + ((((kk >> 2) ^ (r & 7))) << 4) + (kk & 3) * 4);
}
__device__ __forceinline__ float to_tf32(float x) {
  uint32_t u;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
  return __uint_as_float(u);
}
// kind::tf32 instruction descriptor: fp32 accumulate, both operands tf32 and K-major
__device__ __forceinline__ constexpr uint32_t idesc_tf32(int m, int n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[128 x N] (+)= A[128 x KDIM] * B[N x KDIM]^T over images whose base descriptors are adesc0 (128 rows) / bdesc0 (N
// rows); 8 k per MMA. The loop is fully unrolled and a step only adds a compile-time constant to the descriptors'
// address field (the single issuing thread is the critical path of the state-carrying kernel: it must not spend
// its time rebuilding descriptors).
template <int N, int KDIM>
__device__ __forceinline__ void mma_tile(uint32_t tmem_d, uint64_t adesc0, uint64_t bdesc0, bool accumulate) {
  constexpr uint32_t idesc = idesc_tf32(128, N);
#pragma unroll
  for (int ks = 0; ks < KDIM / 8; ++ks) {
    const uint64_t a = adesc0 + (uint64_t)((((ks >> 2) * (128 * 128)) + (ks & 3) * 32) >> 4);
    const uint64_t b = bdesc0 + (uint64_t)((((ks >> 2) * (N * 128)) + (ks & 3) * 32) >> 4);
    umma_tf32(tmem_d, a, b, idesc, (accumulate || ks > 0) ? 1u : 0u);
  }
}
__device__ __forceinline__ uint64_t img_desc(const void* smem_ptr) { return umma_desc_sw128(smem_u32(smem_ptr)); }
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fail(int* err, int code) {
  if (err) atomicCAS(err, 0, code);
}

// ------------------------------------------------------------------------------------------------ chunk-local part
// One CTA = one value head x 128 tokens (two chunks side by side; the cross-chunk blocks of the 128 x 128 products
// are computed and ignored). 256 threads: thread t works on token / TMEM lane t & 127 and, where a row is split, on
// column half t >> 7.
constexpr int PREP_SMEM = 3 * 65536 + 32768 + 2048 + 1024;
constexpr int PREP_THREADS = 256;

// Column `ii` of T = (I + A)^-1 for one 64-token chunk by forward substitution, x_i = [i == ii] - sum_{j<i} A_ij x_j.
// C0 (0 or 32, uniform per warp) is the first column of the warp: x_i = 0 for i < C0, so those rows are skipped.
template <int C0>
__device__ __forceinline__ void solve_column(const float* __restrict__ At, int ii, uint8_t* R0, int row0, int col) {
  float x[64];
#pragma unroll
  for (int i = C0; i < 64; ++i) {
    float a0 = (i == ii) ? 1.f : 0.f, a1 = 0.f;
#pragma unroll
    for (int j = C0; j + 1 < i; j += 2) {
      a0 = fmaf(-At[j * 64 + i], x[j], a0);
      a1 = fmaf(-At[(j + 1) * 64 + i], x[j + 1], a1);
    }
    if ((i - C0) & 1) a0 = fmaf(-At[(i - 1) * 64 + i], x[i - 1], a0);
    x[i] = a0 + a1;
  }
#pragma unroll
  for (int i = C0; i < 64; ++i) *reinterpret_cast<float*>(R0 + img_off(128, row0 + i, col)) = to_tf32(x[i]);
}

__global__ void __launch_bounds__(PREP_THREADS, 1)
gdn_chunk_prep_kernel(const float* __restrict__ qkv, const __nv_bfloat16* __restrict__ proj, int ldp, int off_b, int off_a,
                      const float* __restrict__ A_log, const float* __restrict__ dt_bias, int t0, int tn, int nk, int nv,
                      uint8_t* __restrict__ work, float* __restrict__ gc_out, int n_chunks, int* err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* R0 = smem;                      // K image [128 i][128 d]  -> later T image [128 i][128 j]
  uint8_t* R1 = smem + 65536;              // Q image [128 i][128 d]  -> later scaled K^T image [128 d][128 j]
  uint8_t* R2 = smem + 2 * 65536;          // scaled V^T image [128 v][128 j]
  float* R3 = reinterpret_cast<float*>(smem + 3 * 65536);     // V staging [64][128] (swizzled), then A^T [2][64 j][64 i]
  float* Gs = reinterpret_cast<float*>(smem + 3 * 65536 + 32768);   // [128] cumulative log decay inside the chunk
  float* betas = Gs + 128;                                          // [128]
  float* lgs = betas + 128;                                         // [128] log g
  uint64_t* bar = reinterpret_cast<uint64_t*>(lgs + 128);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 2);

  // (no early launch_dependents here: the dependent scan kernel's CTAs need almost a whole SM each and would only
  // sit on SMs this grid still has tiles for)
  pdl_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row = tid & 127, hf = tid >> 7;
  const int pair = blockIdx.x, vh = blockIdx.y;
  const int kh = vh * nk / nv;
  const int key_dim = nk * KD, conv_dim = 2 * key_dim + nv * VD;
  const int tok0 = pair * 128;             // first token of this tile, relative to t0

  if (tid == 0) {
    mbar_init(&bar[0], 1);
    mbar_init(&bar[1], 1);
    fence_mbar_init();
  }
  __syncwarp();
  if (warp == 0) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  // ---- per-token gates
  if (tid < 128) {
    const int t = tok0 + tid;
    float beta = 0.f, lg = 0.f;
    if (t < tn) {
      const size_t prow = (size_t)(t0 + t) * ldp;
      const float bb = __bfloat162float(proj[prow + off_b + vh]);
      const float aa = __bfloat162float(proj[prow + off_a + vh]) + dt_bias[vh];
      beta = 1.0f / (1.0f + expf(-bb));
      const float sp = aa > 20.f ? aa : log1pf(expf(aa));
      lg = -expf(A_log[vh]) * sp;
    }
    betas[tid] = beta;
    lgs[tid] = lg;
  }
  // ---- q, k rows: l2-normalise (q also / sqrt(kd)), tf32, into the K-major images. A warp owns 16 rows and keeps
  // the loads of eight rows in flight.
#pragma unroll 1
  for (int b = 0; b < 2; ++b) {
    float4 q4[8], k4[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = warp * 16 + b * 8 + u, t = tok0 + i;
      q4[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      k4[u] = q4[u];
      if (t < tn) {
        const float* qrow = qkv + (size_t)(t0 + t) * conv_dim;
        q4[u] = __ldg(reinterpret_cast<const float4*>(qrow + kh * KD + lane * 4));
        k4[u] = __ldg(reinterpret_cast<const float4*>(qrow + key_dim + kh * KD + lane * 4));
      }
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = warp * 16 + b * 8 + u;
      const float qn = warp_sum(q4[u].x * q4[u].x + q4[u].y * q4[u].y + q4[u].z * q4[u].z + q4[u].w * q4[u].w);
      const float kn = warp_sum(k4[u].x * k4[u].x + k4[u].y * k4[u].y + k4[u].z * k4[u].z + k4[u].w * k4[u].w);
      const float qs = rsqrtf(qn + 1e-6f) * rsqrtf((float)KD), ks = rsqrtf(kn + 1e-6f);
      const uint32_t off = img_off(128, i, lane * 4);
      *reinterpret_cast<float4*>(R1 + off) =
          make_float4(to_tf32(q4[u].x * qs), to_tf32(q4[u].y * qs), to_tf32(q4[u].z * qs), to_tf32(q4[u].w * qs));
      *reinterpret_cast<float4*>(R0 + off) =
          make_float4(to_tf32(k4[u].x * ks), to_tf32(k4[u].y * ks), to_tf32(k4[u].z * ks), to_tf32(k4[u].w * ks));
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (tid < 128) {
    const int c0 = tid & ~63;
    float g = 0.f;
    for (int j = c0; j <= tid; ++j) g += lgs[j];
    Gs[tid] = g;
  }
  // ---- (beta V)^T image: rows of V are staged 64 tokens at a time (element (i, v) at [i][v ^ (i & 31)], so both the
  // row-wise writes and the column-wise reads are free of bank conflicts) and re-read transposed
  for (int half = 0; half < 2; ++half) {
    float4 v4[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = half * 64 + warp * 8 + u, t = tok0 + i;
      v4[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (t < tn) v4[u] = __ldg(reinterpret_cast<const float4*>(qkv + (size_t)(t0 + t) * conv_dim + 2 * key_dim + vh * VD + lane * 4));
    }
    __syncthreads();                       // the previous half's staging has been consumed
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int ii = warp * 8 + u, x = ii & 31;
      R3[ii * 128 + ((lane * 4 + 0) ^ x)] = v4[u].x;
      R3[ii * 128 + ((lane * 4 + 1) ^ x)] = v4[u].y;
      R3[ii * 128 + ((lane * 4 + 2) ^ x)] = v4[u].z;
      R3[ii * 128 + ((lane * 4 + 3) ^ x)] = v4[u].w;
    }
    __syncthreads();
    for (int v = warp; v < 128; v += 8) {
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        const int ii = s * 32 + lane, i = half * 64 + ii;
        const float val = R3[ii * 128 + (v ^ (ii & 31))] * betas[i];
        *reinterpret_cast<float*>(R2 + img_off(128, v, i)) = to_tf32(val);
      }
    }
  }
  fence_proxy_async_smem();
  __syncthreads();
  // ---- K K^T and Q K^T (both 128 x 128 x 128)
  if (tid == 0) {
    tc_fence_after();
    mma_tile<128, 128>(tmem_base, img_desc(R0), img_desc(R0), false);
    mma_tile<128, 128>(tmem_base + 128, img_desc(R1), img_desc(R0), false);
    umma_commit(&bar[0]);
  }
  const bool ok0 = mbar_wait(&bar[0], 0);
  if (!ok0) fail(err, VG_ERR_MMA_WAIT);
  tc_fence_after();
  const int chn = row >> 6, ii = row & 63;             // this thread's chunk and row inside it
  const int chunk_id = pair * 2 + chn;
  const bool chunk_live = chunk_id < n_chunks;
  uint8_t* wbase = work + ((size_t)vh * n_chunks + (chunk_live ? chunk_id : 0)) * CHUNK_BYTES;
  const float Gi = Gs[row], bi = betas[row];
  const uint32_t lane_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
  // A^T[chn][j][i] = beta_i e^{G_i - G_j} (k_i . k_j) for j < i; this thread: columns j in [32 hf, 32 hf + 32)
#pragma unroll
  for (int cb = 0; cb < 2; ++cb) {
    uint32_t r[16];
    const int j0 = hf * 32 + cb * 16;
    tmem_ld16(lane_addr + (uint32_t)(chn * 64 + j0), r);
    tmem_ld_wait();
#pragma unroll
    for (int x = 0; x < 16; ++x) {
      const int j = j0 + x;
      const float a = j < ii ? bi * expf(Gi - Gs[chn * 64 + j]) * __uint_as_float(r[x]) : 0.f;
      R3[(chn * 64 + j) * 64 + ii] = a;
    }
  }
  // P[i][j] = e^{G_i - G_j} (q_i . k_j) for j <= i  -> global image (row ii, k j)
#pragma unroll
  for (int cb = 0; cb < 2; ++cb) {
    uint32_t r[16];
    const int j0 = hf * 32 + cb * 16;
    tmem_ld16(lane_addr + (uint32_t)(128 + chn * 64 + j0), r);
    tmem_ld_wait();
    if (chunk_live) {
#pragma unroll
      for (int x4 = 0; x4 < 4; ++x4) {
        float o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = j0 + x4 * 4 + e;
          o[e] = j <= ii ? to_tf32(expf(Gi - Gs[chn * 64 + j]) * __uint_as_float(r[x4 * 4 + e])) : 0.f;
        }
        *reinterpret_cast<float4*>(wbase + WQ_IMG + img_off(CH + KD, ii, j0 + x4 * 4)) = make_float4(o[0], o[1], o[2], o[3]);
      }
    }
  }
  // e^{G_i} Q -> global image (row ii, k d), read back from this thread's row of the Q image (its half of the dims)
  if (chunk_live) {
    const float eg = expf(Gi);
#pragma unroll 4
    for (int d = hf * 64; d < hf * 64 + 64; d += 4) {
      const float4 q4 = *reinterpret_cast<const float4*>(R1 + img_off(128, row, d));
      *reinterpret_cast<float4*>(wbase + img_off(2 * CH, CH + ii, d)) =
          make_float4(to_tf32(q4.x * eg), to_tf32(q4.y * eg), to_tf32(q4.z * eg), to_tf32(q4.w * eg));
    }
  }
  tc_fence_before();
  __syncthreads();                          // R1 (Q image) and both accumulators are free now
  // ---- scaled K^T: shared image (row d, k j) = beta_j e^{G_j} k_j[d]; global image (row d, k jj) = e^{G_C - G_j} k_j[d]
  {
    float sj[4], tj[4];                     // per-token factors of this lane's four tokens
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      const int j = s * 32 + lane;
      sj[s] = betas[j] * expf(Gs[j]);
      tj[s] = expf(Gs[(j >> 6) * 64 + 63] - Gs[j]);
    }
    for (int d = warp; d < 128; d += 8) {
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        const int j = s * 32 + lane;
        const float kv = *reinterpret_cast<const float*>(R0 + img_off(128, j, d));
        *reinterpret_cast<float*>(R1 + img_off(128, d, j)) = to_tf32(sj[s] * kv);
        const int cj = j >> 6;
        if (pair * 2 + cj < n_chunks) {
          uint8_t* wb = work + ((size_t)vh * n_chunks + pair * 2 + cj) * CHUNK_BYTES;
          *reinterpret_cast<float*>(wb + WQ_IMG + img_off(CH + KD, CH + d, j & 63)) = to_tf32(tj[s] * kv);
        }
      }
    }
  }
  __syncthreads();                          // the K image (R0) has been read for the last time
  for (int x = tid; x < 65536 / 16; x += PREP_THREADS) reinterpret_cast<float4*>(R0)[x] = make_float4(0.f, 0.f, 0.f, 0.f);
  __syncthreads();
  // ---- T = (I + A)^-1, one column per thread (threads 0..127)
  if (tid < 128) {
    const float* At = R3 + chn * 64 * 64;
    if ((ii & 32) == 0) solve_column<0>(At, ii, R0, chn * 64, tid);
    else solve_column<32>(At, ii, R0, chn * 64, tid);
  }
  fence_proxy_async_smem();
  __syncthreads();
  // ---- W = T (beta e^G K)  [i][d]   and   U^T = (beta V)^T T^T  [v][i]
  if (tid == 0) {
    tc_fence_after();
    mma_tile<128, 128>(tmem_base, img_desc(R0), img_desc(R1), false);
    mma_tile<128, 128>(tmem_base + 128, img_desc(R2), img_desc(R0), false);
    umma_commit(&bar[1]);
  }
  const bool ok1 = mbar_wait(&bar[1], 0);
  if (!ok1) fail(err, VG_ERR_MMA_WAIT);
  tc_fence_after();
  if (chunk_live) {
#pragma unroll
    for (int cb = 0; cb < 4; ++cb) {         // W row ii of this thread's chunk: its half of the 128 d values
      uint32_t r[16];
      const int d0 = hf * 64 + cb * 16;
      tmem_ld16(lane_addr + (uint32_t)d0, r);
      tmem_ld_wait();
#pragma unroll
      for (int x4 = 0; x4 < 4; ++x4)
        *reinterpret_cast<float4*>(wbase + img_off(2 * CH, ii, d0 + x4 * 4)) =
            make_float4(to_tf32(__uint_as_float(r[x4 * 4])), to_tf32(__uint_as_float(r[x4 * 4 + 1])),
                        to_tf32(__uint_as_float(r[x4 * 4 + 2])), to_tf32(__uint_as_float(r[x4 * 4 + 3])));
    }
  }
  {                                          // U^T row v = row, the 64 tokens of chunk hf (plain fp32 [v][64])
    const bool live = pair * 2 + hf < n_chunks;
    float* ut = reinterpret_cast<float*>(work + ((size_t)vh * n_chunks + (live ? pair * 2 + hf : 0)) * CHUNK_BYTES + WQ_IMG + PK_IMG) + row * CH;
#pragma unroll
    for (int cb = 0; cb < 4; ++cb) {
      uint32_t r[16];
      tmem_ld16(lane_addr + (uint32_t)(128 + hf * 64 + cb * 16), r);
      tmem_ld_wait();
      if (live) {
#pragma unroll
        for (int x4 = 0; x4 < 4; ++x4)
          *reinterpret_cast<float4*>(ut + cb * 16 + x4 * 4) =
              make_float4(__uint_as_float(r[x4 * 4]), __uint_as_float(r[x4 * 4 + 1]), __uint_as_float(r[x4 * 4 + 2]), __uint_as_float(r[x4 * 4 + 3]));
      }
    }
  }
  if (hf == 0 && ii == 63 && chunk_live) gc_out[(size_t)vh * n_chunks + chunk_id] = expf(Gi);
  tc_fence_before();
  __syncthreads();
  pdl_trigger();
  if (warp == 0) tmem_dealloc(tmem_base, 256);
}

// ------------------------------------------------------------------------------------------------ state-carrying part
// One CTA per value head. Warps 0-3: thread v owns row v of S^T (TMEM lane v). Warp 4 lane 0: bulk copies + MMA issue.
// TMEM columns: [ D^T (64) | O^T (64) | S^T (128) ]. The first product of a chunk writes D^T and O^T together
// (B = the stacked W / e^G Q image), the second accumulates onto O^T and S^T together (B = the stacked P / K~^T image);
// S^T is kept pre-multiplied by the next chunk's total decay, so the chunk's outer products are simply accumulated.
constexpr int SCAN_SMEM = 65536 + 32768 + WQ_IMG + PK_IMG + 256 + 1024;

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

__global__ void __launch_bounds__(160, 1)
gdn_chunk_scan_kernel(const uint8_t* __restrict__ work, const float* __restrict__ gc, float* __restrict__ S,
                      const int* __restrict__ in_slot, const int* __restrict__ out_slot, float* __restrict__ o_raw, int t0, int tn,
                      int nv, int n_chunks, int* err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* S0 = smem;                       // S^T image [128 v][128 k]
  uint8_t* DT = S0 + 65536;                 // D^T image [128 v][64 j]
  uint8_t* WQb = DT + 32768;                // [W ; e^G Q] image [128 rows][128 k]
  uint8_t* PKb = WQb + WQ_IMG;              // [P ; K~^T] image  [192 rows][64 j]
  uint64_t* bars = reinterpret_cast<uint64_t*>(PKb + PK_IMG);
  uint64_t* ld_wq = bars, *ld_pk = bars + 1, *mma1 = bars + 2, *mma2 = bars + 3, *thr1 = bars + 4, *thr2 = bars + 5;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  pdl_trigger();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int vh = blockIdx.x;
  if (tid == 0) {
    mbar_init(ld_wq, 1); mbar_init(ld_pk, 1); mbar_init(mma1, 1); mbar_init(mma2, 1);
    mbar_init(thr1, 128); mbar_init(thr2, 128);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 4) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t T_D = tmem_base, T_O = tmem_base + 64, T_S = tmem_base + 128;
  pdl_wait();                               // the images come from the preceding kernel, the state from earlier ones
  const uint8_t* hbase = work + (size_t)vh * n_chunks * CHUNK_BYTES;

  if (warp == 4) {
    if (lane == 0) {
      mbar_arrive_expect_tx(ld_wq, WQ_IMG);
      tma_bulk_g2s(WQb, hbase, WQ_IMG, ld_wq);
      mbar_arrive_expect_tx(ld_pk, PK_IMG);
      tma_bulk_g2s(PKb, hbase + WQ_IMG, PK_IMG, ld_pk);
      const uint64_t d_s0 = img_desc(S0), d_dt = img_desc(DT), d_wq = img_desc(WQb), d_pk = img_desc(PKb);
      for (int c = 0; c < n_chunks; ++c) {
        const uint32_t ph = c & 1;
        if (c + 2 < n_chunks)                                           // pull the chunk after next towards L2
          asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(hbase + (size_t)(c + 2) * CHUNK_BYTES), "r"(CHUNK_BYTES) : "memory");
        if (!mbar_wait(thr2, ph) || !mbar_wait(ld_wq, ph)) { fail(err, VG_ERR_TMA_WAIT); *abort_flag = 1; break; }
        tc_fence_after();
        mma_tile<2 * CH, KD>(T_D, d_s0, d_wq, false);                      // [D^T | O^T] = S^T [W ; e^G Q]^T
        umma_commit(mma1);
        if (!mbar_wait(mma1, ph)) { fail(err, VG_ERR_MMA_WAIT); *abort_flag = 1; break; }
        if (c + 1 < n_chunks) {
          mbar_arrive_expect_tx(ld_wq, WQ_IMG);
          tma_bulk_g2s(WQb, hbase + (size_t)(c + 1) * CHUNK_BYTES, WQ_IMG, ld_wq);
        }
        if (!mbar_wait(thr1, ph) || !mbar_wait(ld_pk, ph)) { fail(err, VG_ERR_TMA_WAIT); *abort_flag = 1; break; }
        tc_fence_after();
        mma_tile<CH + KD, CH>(T_O, d_dt, d_pk, true);                      // [O^T | S^T] += D^T [P ; K~^T]^T
        umma_commit(mma2);
        if (!mbar_wait(mma2, ph)) { fail(err, VG_ERR_MMA_WAIT); *abort_flag = 1; break; }
        if (c + 1 < n_chunks) {
          mbar_arrive_expect_tx(ld_pk, PK_IMG);
          tma_bulk_g2s(PKb, hbase + (size_t)(c + 1) * CHUNK_BYTES + WQ_IMG, PK_IMG, ld_pk);
        }
      }
    }
  } else {
    const int v = tid;                       // 0..127
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    const float* gcp = gc + (size_t)vh * n_chunks;
    // initial state: row v of S^T = column v of S[in_slot]; TMEM gets it times the first chunk's decay
    {
      const float* sp = S + (((size_t)in_slot[t0] * nv + vh) * KD) * VD + v;
      const float g0 = gcp[0];
#pragma unroll 1
      for (int cb = 0; cb < 4; ++cb) {
        uint32_t r[32];
        float sv[32];
#pragma unroll
        for (int x = 0; x < 32; ++x) sv[x] = sp[(size_t)(cb * 32 + x) * VD];
#pragma unroll
        for (int x = 0; x < 32; ++x) r[x] = __float_as_uint(sv[x] * g0);
        tmem_st32(T_S + lane_addr + (uint32_t)(cb * 32), r);
#pragma unroll
        for (int x4 = 0; x4 < 8; ++x4)
          *reinterpret_cast<float4*>(S0 + img_off(128, v, cb * 32 + x4 * 4)) =
              make_float4(to_tf32(sv[x4 * 4]), to_tf32(sv[x4 * 4 + 1]), to_tf32(sv[x4 * 4 + 2]), to_tf32(sv[x4 * 4 + 3]));
      }
      tmem_st_wait();
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(thr2);
    }
    bool dead = false;
    // U^T rows are fetched one chunk ahead (their DRAM latency would otherwise sit on the serial chain)
    const size_t ut_off = (size_t)(WQ_IMG + PK_IMG) + (size_t)v * CH * 4;
    float4 u[16], un[16];
#pragma unroll
    for (int x = 0; x < 16; ++x) un[x] = __ldg(reinterpret_cast<const float4*>(hbase + ut_off) + x);
    float g_n = n_chunks > 1 ? gcp[1] : 1.0f;
    for (int c = 0; c < n_chunks && !dead; ++c) {
      const uint32_t ph = c & 1;
      const bool last = c + 1 == n_chunks;
      const float g_next = last ? 1.0f : g_n;
#pragma unroll
      for (int x = 0; x < 16; ++x) u[x] = un[x];
      if (!last) {
        const float4* utn = reinterpret_cast<const float4*>(hbase + (size_t)(c + 1) * CHUNK_BYTES + ut_off);
#pragma unroll
        for (int x = 0; x < 16; ++x) un[x] = __ldg(utn + x);
        if (c + 2 < n_chunks) g_n = gcp[c + 2];
      }
      if (!mbar_wait(mma1, ph)) { fail(err, VG_ERR_MMA_WAIT); dead = true; break; }
      tc_fence_after();
      // D^T row v = U^T row - S^T W^T row  -> image (row v, k j)
#pragma unroll
      for (int cb = 0; cb < 2; ++cb) {
        uint32_t r[32];
        tmem_ld32(T_D + lane_addr + (uint32_t)(cb * 32), r);
        tmem_ld_wait();
#pragma unroll
        for (int x4 = 0; x4 < 8; ++x4) {
          const float4 uu = u[cb * 8 + x4];
          *reinterpret_cast<float4*>(DT + img_off(128, v, cb * 32 + x4 * 4)) =
              make_float4(to_tf32(uu.x - __uint_as_float(r[x4 * 4])), to_tf32(uu.y - __uint_as_float(r[x4 * 4 + 1])),
                          to_tf32(uu.z - __uint_as_float(r[x4 * 4 + 2])), to_tf32(uu.w - __uint_as_float(r[x4 * 4 + 3])));
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(thr1);
      if (!mbar_wait(mma2, ph)) { fail(err, VG_ERR_MMA_WAIT); dead = true; break; }
      tc_fence_after();
      // raw outputs o[token][vh * VD + v] (the next chunk's first product overwrites O^T, so they are read out first)
#pragma unroll
      for (int cb = 0; cb < 2; ++cb) {
        uint32_t r[32];
        tmem_ld32(T_O + lane_addr + (uint32_t)(cb * 32), r);
        tmem_ld_wait();
#pragma unroll
        for (int x = 0; x < 32; ++x) {
          const int t = c * CH + cb * 32 + x;
          if (t < tn) o_raw[((size_t)(t0 + t) * nv + vh) * VD + v] = __uint_as_float(r[x]);
        }
      }
      // the new state: operand image for the next chunk, and back to TMEM times the next chunk's decay; after the
      // last chunk it goes to the output slot instead
      const int os = last ? out_slot[t0 + tn - 1] : -1;
      float* dp = os >= 0 ? S + (((size_t)os * nv + vh) * KD) * VD + v : nullptr;
#pragma unroll 1
      for (int cb = 0; cb < 4; ++cb) {
        uint32_t r[32];
        tmem_ld32(T_S + lane_addr + (uint32_t)(cb * 32), r);
        tmem_ld_wait();
        if (!last) {
#pragma unroll
          for (int x4 = 0; x4 < 8; ++x4)
            *reinterpret_cast<float4*>(S0 + img_off(128, v, cb * 32 + x4 * 4)) =
                make_float4(to_tf32(__uint_as_float(r[x4 * 4])), to_tf32(__uint_as_float(r[x4 * 4 + 1])),
                            to_tf32(__uint_as_float(r[x4 * 4 + 2])), to_tf32(__uint_as_float(r[x4 * 4 + 3])));
        } else if (dp) {
#pragma unroll
          for (int x = 0; x < 32; ++x) dp[(size_t)(cb * 32 + x) * VD] = __uint_as_float(r[x]);
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(thr2);
      // off the serial chain (the next chunk's first products only read the image): the accumulator copy of the
      // state times the next chunk's decay, needed by the next chunk's LAST product
      if (!last) {
#pragma unroll 1
        for (int cb = 0; cb < 4; ++cb) {
          uint32_t r[32];
          tmem_ld32(T_S + lane_addr + (uint32_t)(cb * 32), r);
          tmem_ld_wait();
#pragma unroll
          for (int x = 0; x < 32; ++x) r[x] = __float_as_uint(__uint_as_float(r[x]) * g_next);
          tmem_st32(T_S + lane_addr + (uint32_t)(cb * 32), r);
        }
        tmem_st_wait();
      }
    }
  }
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem_base, 256);
}

}  // namespace

extern "C" long long vg_gdn_chunk_work_bytes(int tn, int nv) {
  const long long n_chunks = (tn + CH - 1) / CH;
  return n_chunks * nv * (long long)CHUNK_BYTES + n_chunks * nv * 4 + 1024;
}

int vg_gdn_out_norm_launch(const float* o_raw, const void* proj, int ldp, int off_z, const float* norm_w, int t0, int tn,
                           void* out_f16, int nv, int vd, float eps, cudaStream_t st);

// One linear chain of `tn` columns starting at column t0 (prefill) in chunked form: the carried state is read from
// slot in_slot[t0] and, when out_slot[t0 + tn - 1] >= 0, written there after the last token. `work` is scratch of
// vg_gdn_chunk_work_bytes(tn, nv) bytes (1024-byte aligned), `o_raw` fp32 scratch of (t0 + tn) * nv * vd elements.
extern "C" int vg_gdn_chunk_prefill(const float* qkv, const void* proj, int ldp, int off_z, int off_b, int off_a, float* S,
                                    const float* A_log, const float* dt_bias, const float* norm_w, int t0, int tn,
                                    const int* in_slot, const int* out_slot, void* out_f16, int nk, int nv, int kd, int vd,
                                    float eps, void* work, float* o_raw, int* err, cudaStream_t st) {
  if (tn <= 0) return 0;
  if (kd != KD || vd != VD) return -3;
  const int key_dim = nk * KD, conv_dim = 2 * key_dim + nv * VD;
  if ((reinterpret_cast<uintptr_t>(qkv) & 15) || (conv_dim % 4) != 0 || (reinterpret_cast<uintptr_t>(work) & 1023) || !o_raw) return -2;
  const int n_chunks = (tn + CH - 1) / CH, n_pairs = (n_chunks + 1) / 2;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gdn_chunk_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PREP_SMEM);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gdn_chunk_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SCAN_SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  uint8_t* wk = static_cast<uint8_t*>(work);
  float* gc = reinterpret_cast<float*>(wk + (size_t)n_chunks * nv * CHUNK_BYTES);
  cudaError_t e = launch_pdl(gdn_chunk_prep_kernel, dim3(n_pairs, nv), dim3(PREP_THREADS), PREP_SMEM, st, qkv,
                             static_cast<const __nv_bfloat16*>(proj), ldp, off_b, off_a, A_log, dt_bias, t0, tn, nk, nv, wk, gc,
                             n_chunks, err);
  if (e != cudaSuccess) return (int)e;
  e = launch_pdl(gdn_chunk_scan_kernel, dim3(nv), dim3(160), SCAN_SMEM, st, (const uint8_t*)wk, (const float*)gc, S, in_slot,
                 out_slot, o_raw, t0, tn, nv, n_chunks, err);
  if (e != cudaSuccess) return (int)e;
  return vg_gdn_out_norm_launch(o_raw, proj, ldp, off_z, norm_w, t0, tn, out_f16, nv, vd, eps, st);
}

// Decode / verify GEMM on the block-scaled FP4 tensor-core path (tcgen05.mma kind::mxf4nvf4, sm_100a).
//
//   Y[n, m] = row_scale[m] * sum_k nvfp4(W[m, k]) * X[n, k],   N <= 16
//
// The f16 path (gemm_tc.cu) retires one M128 x N16 x K16 MMA per ~106 cycles per SM, which caps a 4-bit
// weight stream at about 3 TB/s. Here one instruction covers K = 64 and the packed e2m1 weights and their
// e4m3 block scales are consumed straight from shared memory / TMEM with no dequantisation work at all.
// The hardware needs both operands in FP4, so each activation column is expanded into a four-term NVFP4
// residual series  x ~ x0 + x1 + x2 + x3  (term t quantises what terms < t left over, with a fixed global
// scale ratio of 1/8 between terms); the four terms of the 16 columns form the 64 rows of the B operand,
// one MMA multiplies the weights with all of them, and the epilogue recombines
//   y = g0[n] * (D0 + D1/8 + D2/64 + D3/512).
// Four e2m1 terms carry ~10 bits of each 16-element block's range, i.e. the activation precision of the
// 16-bit path; weights are exact. Every column is quantised on its own and MMA columns are independent, so
// the result of a column does not depend on the batch width.
//
// CTA (256 threads): warp 0 weight producer (bulk copies of pre-tiled 128 x 256 slabs: 16 KB packed values
// in the UMMA 128-byte-swizzle layout + 2 KB scales in the scale-factor chunk layout), warp 1 activation
// producer (tensor copy of the 64 x 256 B tile + bulk copy of its scale chunks), warps 2-3 MMA issuers
// (even / odd slabs, separate accumulators; each copies its slab's scale factors to TMEM with tcgen05.cp and
// issues four K=64 MMAs), warps 4-7 epilogue. Split-K over a thread-block cluster with a rank-order DSMEM
// reduction, exactly as in gemm_tc.cu. All waits are bounded.
#include <cuda.h>
#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"
#include "api.h"

namespace {
using namespace vg;

constexpr int BM = 128;
constexpr int BKQ = 256;                    // K elements per slab
constexpr int NT = 64;                      // B rows: 4 terms x 16 columns
constexpr int TERMS = 4;
constexpr int A_BYTES = BM * BKQ / 2;       // 16384
constexpr int SF_BYTES = 4 * 512;           // scale chunks of one slab (4 K=64 steps)
constexpr int B_BYTES = NT * BKQ / 2;       // 8192
constexpr int STAGE = A_BYTES + SF_BYTES + B_BYTES + SF_BYTES;   // 28672
constexpr int NS = 6;                       // stages (even: one issuer per stage)
constexpr int THREADS = 256;
constexpr uint32_t ACC_W = 64;              // columns of one accumulator
constexpr uint32_t SF_COLS = 32;            // TMEM columns of one slab's scale factors (A: 16, B: 16)
constexpr uint32_t TMEM_COLS = 256;         // 2 accumulators + 2 issuers x 2 scale buffers

struct Fp4Params {
  const uint8_t* wt;          // [MT][KS][A_BYTES + SF_BYTES]
  const float* row_scale;
  const uint8_t* sfb;         // [KS][SF_BYTES] activation scale chunks
  const float* g0;            // [16] per-column global scale of term 0
  void* out;
  int M, N, ldo, ks_total, out_f32;
  int* err;
  int ar;
  // grouped (MoE decode) mode: blockIdx.y = work item; the item's expert picks the weight tiles, its pair index
  // picks the activation column (pair / x_div) and the output row (pair)
  int grouped, tiles_per_expert, x_div;
  const int* g_exp;
  const int* g_off;
  int has_conv;
  VgConvEpi conv;
  VgCommCtx comm;
};

constexpr int smem_total(int ns) { return ns * STAGE + (2 * ns + 1) * 8 + 16 + 1024; }
constexpr int SMEM_TOTAL = smem_total(NS);
constexpr int CONV_MAX_CK = 4;            // taps the fused conv epilogue supports
constexpr int CONV_SMEM = 16 * (CONV_MAX_CK - 1) * BM * 4;   // prefetched state samples, appended after SMEM_TOTAL
constexpr int SPLITK_PUSH_MAX = CONV_MAX_CK;                 // split-K widths whose partial slots fit the same region

// instruction descriptor for kind::mxf4nvf4, e2m1 x e2m1, ue4m3 scales, K = 64, both operands K-major
__device__ __forceinline__ constexpr uint32_t idesc_fp4(int m, int n) {
  return (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | (0u << 23) | ((uint32_t)(m >> 4) << 24);
}
// shared-memory descriptor of a 32 x 16-byte scale chunk (no swizzle: 8-row groups are 128 bytes apart)
__device__ __forceinline__ uint64_t sf_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)(16 >> 4) << 16;        // leading byte offset (one 16-byte column only)
  d |= (uint64_t)(128 >> 4) << 32;       // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;
  return d;
}
__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void umma_fp4(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa,
                                         uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void fail(int* err, int code, volatile int* abort_flag) {
  if (err) atomicCAS(err, 0, code);
  *abort_flag = 1;
}

// NSK: ring stages. Six for the dense layers (one CTA per SM, deep prefetch); two for the grouped MoE form, whose
// work items are short (K / 256 slabs of one expert) and numerous, so two CTAs share an SM.
template <int NSK>
__global__ void __launch_bounds__(THREADS, NSK <= 2 ? 2 : 1)
gemm_fp4_kernel(const Fp4Params p, const __grid_constant__ CUtensorMap tmap_b) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + NSK * STAGE);
  uint64_t* full = bars;                 // both producers arrive (count 2) + their bytes
  uint64_t* empty = full + NSK;           // MMA commit
  uint64_t* acc_full = empty + NSK;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int mt = blockIdx.x;
  int b_tile = 0, b_col = 0, out_row = 0;
  if (p.grouped) {
    pdl_wait();                            // the group tables come from the router kernel
    const int e = p.g_exp[blockIdx.y];
    if (e < 0) return;                     // expert not resident on this rank (uniform for the CTA)
    out_row = p.g_off[blockIdx.y];
    const int src = out_row / p.x_div;     // activation row the pair reads
    b_tile = src >> 4;
    b_col = src & 15;
    mt = e * p.tiles_per_expert + (int)blockIdx.x;
  }
  const int S = gridDim.z, z = blockIdx.z;
  const int ks0 = (int)(((long long)z * p.ks_total) / S);
  const int ks1 = (int)(((long long)(z + 1) * p.ks_total) / S);
  const int nks = ks1 - ks0;
  const int rot = nks > 0 ? (int)(((unsigned)mt * 7u + (unsigned)z * 3u) % (unsigned)nks) : 0;
  auto slab_of = [&](int i) { int k = i + rot; return ks0 + (k >= nks ? k - nks : k); };
  if (threadIdx.x == 0) trace(4 * 16);
  pdl_trigger();
  const bool splitk_push = S > 1 && S <= SPLITK_PUSH_MAX && !p.has_conv;
  if (splitk_push) cluster_arrive_relaxed();   // waited for just before the partial columns are pushed to the leader

  if (threadIdx.x == 0) {
    for (int i = 0; i < NSK; ++i) { mbar_init(&full[i], 2); mbar_init(&empty[i], 1); }
    mbar_init(acc_full, 2);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) trace(4 * 16 + 5);

  if (warp == 0) {
    if (lane == 0) {
      // Weights do not depend on the preceding kernel: the ring fills before that kernel has finished (the
      // activation producer and the epilogue do the waiting). Asking L2 for further slabs ahead of time with
      // bulk prefetches measured slower at every depth, so only the ring runs ahead.
      const uint8_t* wbase = p.wt + (size_t)mt * p.ks_total * (A_BYTES + SF_BYTES);
      for (int i = 0; i < nks && !*abort_flag; ++i) {
        const int s = i % NSK;
        if (!mbar_wait(&empty[s], ((i / NSK) & 1) ^ 1)) { fail(p.err, VG_ERR_EMPTY_WAIT, abort_flag); break; }
        uint8_t* st = smem + (size_t)s * STAGE;
        mbar_arrive_expect_tx(&full[s], A_BYTES + SF_BYTES);
        tma_bulk_g2s(st, wbase + (size_t)slab_of(i) * (A_BYTES + SF_BYTES), A_BYTES + SF_BYTES, &full[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      pdl_wait();                          // the activation series comes from the preceding kernel
      trace(4 * 16 + 1);
      for (int i = 0; i < nks && !*abort_flag; ++i) {
        const int s = i % NSK;
        if (!mbar_wait(&empty[s], ((i / NSK) & 1) ^ 1)) { fail(p.err, VG_ERR_EMPTY_WAIT, abort_flag); break; }
        uint8_t* st = smem + (size_t)s * STAGE + A_BYTES + SF_BYTES;
        const int ks = slab_of(i);
        mbar_arrive_expect_tx(&full[s], B_BYTES + SF_BYTES);
        tma_tensor2d_g2s(st, &tmap_b, ks * (BKQ / 2), b_tile * NT, &full[s]);
        tma_bulk_g2s(st + B_BYTES, p.sfb + ((size_t)b_tile * p.ks_total + ks) * SF_BYTES, SF_BYTES, &full[s]);
      }
    }
  } else if (warp == 2 || warp == 3) {
    if (lane == 0) {
      const int me = warp - 2;
      const uint32_t idesc = idesc_fp4(BM, NT);
      const uint32_t tmem_acc = tmem_base + (uint32_t)me * ACC_W;
      const uint32_t tmem_sf0 = tmem_base + 2 * ACC_W + (uint32_t)me * 2 * SF_COLS;
      bool ok = true;
      int mine = 0;
      for (int i = me; i < nks && !*abort_flag; i += 2, ++mine) {
        const int s = i % NSK;
        if (!mbar_wait(&full[s], (i / NSK) & 1)) { fail(p.err, VG_ERR_TMA_WAIT, abort_flag); ok = false; break; }
        if (i == 0) trace(4 * 16 + 3);
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + (size_t)s * STAGE);
        const uint32_t sfa_addr = a_addr + A_BYTES;
        const uint32_t b_addr = sfa_addr + SF_BYTES;
        const uint32_t sfb_addr = b_addr + B_BYTES;
        const uint32_t sf_t = tmem_sf0 + (uint32_t)(mine & 1) * SF_COLS;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          tmem_cp_sf(sf_t + 4 * j, sf_desc(sfa_addr + 512 * j));
          tmem_cp_sf(sf_t + 16 + 4 * j, sf_desc(sfb_addr + 512 * j));
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          umma_fp4(tmem_acc, umma_desc_sw128(a_addr + 32 * j), umma_desc_sw128(b_addr + 32 * j), idesc, sf_t + 4 * j,
                   sf_t + 16 + 4 * j, (i >= 2 || j != 0) ? 1u : 0u);
        }
        umma_commit(&empty[s]);
      }
      if (ok) umma_commit(acc_full);
    }
  }
  __syncwarp();

  // ---------------------------------------------------------------- epilogue: warps 4..7, thread = weight row
  const bool epi = warp >= 4;
  const int q = warp & 3;
  const int m_local = q * 32 + lane;
  float y[16];
  bool have = false;
  uint32_t ar_epoch = 0;
  // fused conv: state samples and taps of this thread's channel, fetched while the main loop runs
  const bool conv_row = epi && p.has_conv && mt * BM + m_local < p.conv.conv_dim && z == 0;
  float* conv_pre = reinterpret_cast<float*>(smem + smem_total(NSK) - 1024);      // [16][CONV_MAX_CK - 1][BM]
  float wk[CONV_MAX_CK];
  uint32_t n_state = 0;                    // 2 bits per column: samples that come from the rolling state
  // The per-row weight scale and the columns' global scales are fetched while the main loop runs (the row scale is
  // a weight: before the dependency wait), so the epilogue's stores do not start with two global round trips.
  __shared__ float g0s[16];
  float rsc_pre = 1.0f;
  if (epi && p.row_scale) {
    const int m_pre = mt * BM + m_local;
    if (p.grouped ? (int)blockIdx.x * BM + m_local < p.M : m_pre < p.M) rsc_pre = p.row_scale[m_pre];
  }
  if (epi) {
    pdl_wait();                            // before g0 / epoch reads and every output write
    ar_epoch = p.ar ? *p.comm.epoch + 1 : 0;
    if (threadIdx.x - 128 < 16) g0s[threadIdx.x - 128] = p.g0[b_tile * 16 + (threadIdx.x - 128)];
    if (conv_row) {
      const VgConvEpi& cv = p.conv;
      const int ck = cv.ck, ch = mt * BM + m_local;
#pragma unroll
      for (int i = 0; i < CONV_MAX_CK; ++i) wk[i] = i < ck ? cv.w[(size_t)ch * ck + i] : 0.f;
      for (int t = 0; t < p.N; ++t) {
        int cur = t, j = ck - 1;
        for (; j >= 0 && cur >= 0; --j) cur = cv.parent[cur];
        const int d = ck - 1 - j;
        const float* st = cv.state + ((size_t)cv.in_slot[t] * cv.conv_dim + ch) * ck;
        for (int jj = j; jj >= 0; --jj) conv_pre[(t * (CONV_MAX_CK - 1) + jj) * BM + m_local] = st[jj + d];
        n_state |= (uint32_t)(j + 1) << (2 * t);
      }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");          // g0s visible to the four epilogue warps
    if (mbar_wait(acc_full, 0)) {
      if (threadIdx.x == 128) trace(4 * 16 + 4);
      tc_fence_after();
#pragma unroll
      for (int n = 0; n < 16; ++n) y[n] = 0.f;
      const float tw[TERMS] = {1.0f, 0.125f, 0.015625f, 0.001953125f};
#pragma unroll
      for (int t = 0; t < TERMS; ++t) {
        uint32_t a0[16], a1[16];
        tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(t * 16), a0);
        tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + ACC_W + (uint32_t)(t * 16), a1);
        tmem_ld_wait();
#pragma unroll
        for (int n = 0; n < 16; ++n) {
          const float d = nks >= 2 ? __uint_as_float(a0[n]) + __uint_as_float(a1[n]) : __uint_as_float(a0[n]);
          y[n] = fmaf(d, tw[t], y[n]);
        }
      }
      have = true;
      if (threadIdx.x == 128) trace(4 * 16 + 8);
    } else {
      fail(p.err, VG_ERR_MMA_WAIT, abort_flag);
    }
  }
  if (splitk_push) {
    // Split-K reduction, push form: the other CTAs of the cluster store their partial columns into slots of the
    // leader's shared memory (a region no pipeline stage uses, so a fast peer cannot disturb the leader's running
    // MMAs); one cluster barrier orders the stores before the leader's reads, which are local and in rank order.
    float* slots = conv_pre;                               // [S - 1][16][BM] in the leader; conv launches never come here
    cluster_wait();                                        // pairs with the arrive at entry: the leader has started
    if (z != 0 && epi && have) {
      const uint32_t dst = dsmem_map(smem_u32(slots + (size_t)(z - 1) * 16 * BM), 0u);
#pragma unroll
      for (int n = 0; n < 16; ++n)
        if (n < p.N) dsmem_st_f32(dst + (uint32_t)((n * BM + m_local) * 4), y[n]);
    }
    cluster_sync_all();
    if (threadIdx.x == 128) trace(4 * 16 + 9);
    if (z == 0 && epi && have) {
      for (int s2 = 1; s2 < S; ++s2) {
        const float* sl = slots + (size_t)(s2 - 1) * 16 * BM;
#pragma unroll
        for (int n = 0; n < 16; ++n)
          if (n < p.N) y[n] += sl[n * BM + m_local];
      }
    }
    if (threadIdx.x == 128) trace(4 * 16 + 10);
  } else if (S > 1) {
    float* red = reinterpret_cast<float*>(smem);          // stage 0 is idle once every MMA has completed
    if (epi && have) {
#pragma unroll
      for (int n = 0; n < 16; ++n)
        if (n < p.N) red[n * BM + m_local] = y[n];
    }
    cluster_sync_all();
    if (threadIdx.x == 128) trace(4 * 16 + 9);
    if (z == 0 && epi && have) {
      const uint32_t red_addr = smem_u32(red);
      for (int s = 1; s < S; ++s) {
        const uint32_t remote = dsmem_map(red_addr, (uint32_t)s);
#pragma unroll
        for (int n = 0; n < 16; ++n)                       // only the columns that exist cross the cluster
          if (n < p.N) y[n] += dsmem_ld_f32(remote + (uint32_t)((n * BM + m_local) * 4));
      }
    }
    cluster_sync_all();
    if (threadIdx.x == 128) trace(4 * 16 + 10);
  }
  const int m = mt * BM + m_local;
  if (epi && z == 0 && p.ar) {
    // fused tensor-parallel all-reduce (same protocol as gemm_tc.cu)
    __shared__ int ar_failed;
    const VgCommCtx& c = p.comm;
    const uint32_t e = ar_epoch;
    const int set = e & 1;
    const int et = threadIdx.x - 128;
    const float rsc = rsc_pre;
    if (et == 0) ar_failed = 0;
    if (p.ar != 2 && have && m < p.M) {
      for (int k = 0; k < c.world; ++k) {
        const int peer = (c.rank + k) % c.world;
        float* dst = reinterpret_cast<float*>(c.data[peer] + c.slots_off + (size_t)(set * MAX_RANKS + c.rank) * c.slot_bytes);
#pragma unroll
        for (int n = 0; n < 16; ++n)
          if (n < p.N) dst[(size_t)n * p.M + m] = y[n] * g0s[n] * rsc;
      }
    }
    if (p.ar == 3) {
      // In-switch reduction: the partial rows stay in this rank's own copy of the multimem slot (plain local
      // stores, nothing crosses NVLink here). Each CTA then publishes the epoch of its 128-row tile on every rank
      // with one multicast store; the consumer (add_rmsnorm_fp4_kernel<2>) waits per tile for all W ranks' words and
      // reads each element once with multimem.ld_reduce, the switch adding the W copies.
      if (have && m < p.M) {
        float* dst = reinterpret_cast<float*>(c.data[c.rank] + c.mm_off + (size_t)set * c.mm_slot_bytes);
#pragma unroll
        for (int n = 0; n < 16; ++n)
          if (n < p.N) dst[(size_t)n * p.M + m] = y[n] * g0s[n] * rsc;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (et == 0) {
        asm volatile("fence.acq_rel.sys;" ::: "memory");   // release: the tile's rows are visible system-wide before its word is
        multimem_st_u32(c.mc + c.mmflags_off + ((size_t)(set * MAX_CTAS + (int)blockIdx.x) * MAX_RANKS + c.rank) * 4, e);
        trace(4 * 16 + 6);
      }
    } else if (p.ar == 2) {
      // Publish only: every value goes to every rank's receive slot (this rank's own included) as an 8-byte
      // (value, epoch) pair: one store each, no fence and no flag lines. The residual-add / RMSNorm kernel that
      // follows polls its own memory, takes a pair once its epoch matches and sums in rank order.
      if (have && m < p.M) {
        for (int k = 0; k < c.world; ++k) {
          const int peer = (c.rank + k) % c.world;
          uint2* dst = reinterpret_cast<uint2*>(c.data[peer] + c.slots_off + (size_t)(set * MAX_RANKS + c.rank) * c.slot_bytes);
#pragma unroll
          for (int n = 0; n < 16; ++n)
            if (n < p.N) {
              const uint32_t bits = __float_as_uint(y[n] * g0s[n] * rsc);
              asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(dst + (size_t)n * p.M + m), "r"(bits), "r"(e) : "memory");
            }
        }
      }
      if (et == 0) trace(4 * 16 + 6);
    } else {
    __threadfence_system();
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (et == 0) trace(4 * 16 + 6);
    if (et < c.world)
      st_release_sys(reinterpret_cast<uint32_t*>(c.data[et] + c.flags_off) + flag_index(set, c.rank, (int)blockIdx.x), e);
    if (et < c.world) {
      const uint32_t* f = reinterpret_cast<const uint32_t*>(c.data[c.rank] + c.flags_off) + flag_index(set, et, (int)blockIdx.x);
      if (!wait_flag(f, e, c.timeout_ns)) { atomicCAS(c.status, 0, VG_ERR_PEER_WAIT); ar_failed = 1; }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (et == 0) trace(4 * 16 + 7);
    if (!ar_failed && have && m < p.M) {
      const float* base = reinterpret_cast<const float*>(c.data[c.rank] + c.slots_off + (size_t)set * MAX_RANKS * c.slot_bytes);
      const size_t stride = c.slot_bytes / sizeof(float);
#pragma unroll
      for (int n = 0; n < 16; ++n) {
        if (n < p.N) {
          const size_t idx = (size_t)n * p.M + m;
          float sum = 0.f;
          for (int q2 = 0; q2 < c.world; ++q2) sum += __ldcg(&base[(size_t)q2 * stride + idx]);
          if (p.out_f32) reinterpret_cast<float*>(p.out)[(size_t)n * p.ldo + m] = sum;
          else reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)n * p.ldo + m] = __float2bfloat16_rn(sum);
        }
      }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (et == 0) {
      __threadfence();
      if (atomicAdd(c.done_ctr, 1u) == gridDim.x - 1) { *c.done_ctr = 0; *c.epoch = e; }
    }
    }
  } else if (p.grouped) {
    const int mi = (int)blockIdx.x * BM + m_local;          // row inside the expert
    if (epi && have && z == 0 && mi < p.M) {
      float yv = 0.f;
#pragma unroll
      for (int n = 0; n < 16; ++n) yv = n == b_col ? y[n] : yv;
      const float v = yv * g0s[b_col] * rsc_pre;
      if (p.out_f32) reinterpret_cast<float*>(p.out)[(size_t)out_row * p.ldo + mi] = v;
      else reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)out_row * p.ldo + mi] = __float2bfloat16_rn(v);
    }
  } else if (epi && have && z == 0 && m < p.M) {
    const float rsc = rsc_pre;
    float* xs = reinterpret_cast<float*>(smem) + 16 * BM;     // second half of idle stage 0: [n][row] samples
#pragma unroll
    for (int n = 0; n < 16; ++n) {
      if (n < p.N) {
        const float v = y[n] * g0s[n] * rsc;
        if (p.out_f32) reinterpret_cast<float*>(p.out)[(size_t)n * p.ldo + m] = v;
        else reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)n * p.ldo + m] = __float2bfloat16_rn(v);
        if (conv_row) xs[n * BM + m_local] = __bfloat162float(__float2bfloat16_rn(v));   // what a reader of `out` sees
      }
    }
    if (conv_row) {
      // Depthwise causal conv + SiLU of this channel for every column, then the state update. Only this thread
      // touches the channel, so computing every output before any state write needs no barrier.
      const VgConvEpi& cv = p.conv;
      const int ck = cv.ck;
      for (int pass = 0; pass < 2; ++pass) {
        for (int t = 0; t < p.N; ++t) {
          const int os = cv.out_slot[t];
          if (pass == 1 && os < 0) continue;
          float win[CONV_MAX_CK];
          const int ns = (int)((n_state >> (2 * t)) & 3u);
          int cur = t;
          for (int j = ck - 1; j >= ns; --j) {
            win[j] = xs[cur * BM + m_local];
            cur = cv.parent[cur];
          }
          for (int jj = 0; jj < ns; ++jj) win[jj] = conv_pre[(t * (CONV_MAX_CK - 1) + jj) * BM + m_local];
          if (pass == 0) {
            float acc = 0.f;
            for (int i = 0; i < ck; ++i) acc = fmaf(wk[i], win[i], acc);
            cv.out[(size_t)t * cv.conv_dim + m] = silu(acc);
          } else {
            float* dst = cv.state + ((size_t)os * cv.conv_dim + m) * ck;
            for (int i = 0; i < ck; ++i) dst[i] = win[i];
          }
        }
      }
    }
  }
  if (threadIdx.x == 128) trace(4 * 16 + 11);
  if (*abort_flag && threadIdx.x == 0) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) trace(4 * 16 + 2);
  if (warp == 2) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ------------------------------------------------------------------ persistent variant
// For weights with more 128-row tiles than SMs (gate_up, LM head): one CTA per SM walks its tiles
// (blockIdx.x, blockIdx.x + gridDim.x, ...) with the ring running straight through tile boundaries, so there is
// no drain / refill between tiles and no ragged last wave of cold CTAs. Accumulators are double-buffered in
// TMEM (2 tiles x 2 issuers): the epilogue of tile i overlaps the main loop of tile i + 1. Plain epilogue only
// (no split-K, fused all-reduce or conv); needs at least two slabs per tile.
constexpr uint32_t P_TMEM_COLS = 512;      // 4 accumulators (cols 0..255) + 2 issuers x 2 scale buffers (256..383)
constexpr int P_SMEM_TOTAL = NS * STAGE + (2 * NS + 4) * 8 + 16 + 1024;

__global__ void __launch_bounds__(THREADS, 1)
gemm_fp4_persist_kernel(const Fp4Params p, const __grid_constant__ CUtensorMap tmap_b, int tiles) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + NS * STAGE);
  uint64_t* empty = full + NS;
  uint64_t* acc_full = empty + NS;       // [2] both issuers commit
  uint64_t* acc_empty = acc_full + 2;    // [2] one arrival per epilogue warp
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nks = p.ks_total;
  const int nt = ((int)blockIdx.x < tiles) ? (tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
  const int total = nt * nks;
  if (threadIdx.x == 0) trace(4 * 16);
  pdl_trigger();

  if (threadIdx.x == 0) {
    for (int i = 0; i < NS; ++i) { mbar_init(&full[i], 2); mbar_init(&empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 2); mbar_init(&acc_empty[i], 4); }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, P_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int ti = 0, sl = 0;
      for (int it = 0; it < total && !*abort_flag; ++it) {
        const int mt = (int)blockIdx.x + ti * (int)gridDim.x;
        const int rot = (int)(((unsigned)mt * 7u) % (unsigned)nks);
        const int ks = sl + rot >= nks ? sl + rot - nks : sl + rot;
        const int s = it % NS;
        if (!mbar_wait(&empty[s], ((it / NS) & 1) ^ 1)) { fail(p.err, VG_ERR_EMPTY_WAIT, abort_flag); break; }
        mbar_arrive_expect_tx(&full[s], A_BYTES + SF_BYTES);
        tma_bulk_g2s(smem + (size_t)s * STAGE, p.wt + ((size_t)mt * nks + ks) * (A_BYTES + SF_BYTES), A_BYTES + SF_BYTES,
                     &full[s]);
        if (++sl == nks) { sl = 0; ++ti; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      pdl_wait();                          // the activation series comes from the preceding kernel
      trace(4 * 16 + 1);
      int ti = 0, sl = 0;
      for (int it = 0; it < total && !*abort_flag; ++it) {
        const int mt = (int)blockIdx.x + ti * (int)gridDim.x;
        const int rot = (int)(((unsigned)mt * 7u) % (unsigned)nks);
        const int ks = sl + rot >= nks ? sl + rot - nks : sl + rot;
        const int s = it % NS;
        if (!mbar_wait(&empty[s], ((it / NS) & 1) ^ 1)) { fail(p.err, VG_ERR_EMPTY_WAIT, abort_flag); break; }
        uint8_t* st = smem + (size_t)s * STAGE + A_BYTES + SF_BYTES;
        mbar_arrive_expect_tx(&full[s], B_BYTES + SF_BYTES);
        tma_tensor2d_g2s(st, &tmap_b, ks * (BKQ / 2), 0, &full[s]);
        tma_bulk_g2s(st + B_BYTES, p.sfb + (size_t)ks * SF_BYTES, SF_BYTES, &full[s]);
        if (++sl == nks) { sl = 0; ++ti; }
      }
    }
  } else if (warp == 2 || warp == 3) {
    if (lane == 0) {
      const int me = warp - 2;
      const uint32_t idesc = idesc_fp4(BM, NT);
      const uint32_t tmem_sf0 = tmem_base + 4 * ACC_W + (uint32_t)me * 2 * SF_COLS;
      int mine = 0;
      for (int it = me; it < total && !*abort_flag; it += 2, ++mine) {
        const int ti = it / nks, sl = it - ti * nks;
        const int buf = ti & 1;
        const uint32_t tmem_acc = tmem_base + (uint32_t)(buf * 2 + me) * ACC_W;
        if (sl < 2) {
          // first slab of this issuer in the tile: the epilogue must have drained the buffer (two tiles ago)
          if (!mbar_wait(&acc_empty[buf], (((ti >> 1) & 1) ^ 1))) { fail(p.err, VG_ERR_MMA_WAIT, abort_flag); break; }
          tc_fence_after();
        }
        const int s = it % NS;
        if (!mbar_wait(&full[s], (it / NS) & 1)) { fail(p.err, VG_ERR_TMA_WAIT, abort_flag); break; }
        if (it == 0) trace(4 * 16 + 3);
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + (size_t)s * STAGE);
        const uint32_t sfa_addr = a_addr + A_BYTES;
        const uint32_t b_addr = sfa_addr + SF_BYTES;
        const uint32_t sfb_addr = b_addr + B_BYTES;
        const uint32_t sf_t = tmem_sf0 + (uint32_t)(mine & 1) * SF_COLS;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          tmem_cp_sf(sf_t + 4 * j, sf_desc(sfa_addr + 512 * j));
          tmem_cp_sf(sf_t + 16 + 4 * j, sf_desc(sfb_addr + 512 * j));
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          umma_fp4(tmem_acc, umma_desc_sw128(a_addr + 32 * j), umma_desc_sw128(b_addr + 32 * j), idesc, sf_t + 4 * j,
                   sf_t + 16 + 4 * j, (sl >= 2 || j != 0) ? 1u : 0u);
        }
        umma_commit(&empty[s]);
        if (sl >= nks - 2) umma_commit(&acc_full[buf]);      // this issuer's last slab of the tile
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps 4..7, thread = weight row
    const int q = warp & 3;
    const int m_local = q * 32 + lane;
    pdl_wait();                            // before g0 reads and every output write
    float g0r[16];
#pragma unroll
    for (int n = 0; n < 16; ++n) g0r[n] = n < p.N ? p.g0[n] : 0.f;
    const float tw[TERMS] = {1.0f, 0.125f, 0.015625f, 0.001953125f};
    for (int ti = 0; ti < nt && !*abort_flag; ++ti) {
      const int buf = ti & 1;
      const int mt = (int)blockIdx.x + ti * (int)gridDim.x;
      const int m = mt * BM + m_local;
      const float rsc = (p.row_scale && m < p.M) ? p.row_scale[m] : 1.0f;
      if (!mbar_wait(&acc_full[buf], (ti >> 1) & 1)) { fail(p.err, VG_ERR_MMA_WAIT, abort_flag); break; }
      if (threadIdx.x == 128 && ti == 0) trace(4 * 16 + 4);
      tc_fence_after();
      float y[16];
#pragma unroll
      for (int n = 0; n < 16; ++n) y[n] = 0.f;
#pragma unroll
      for (int t = 0; t < TERMS; ++t) {
        uint32_t a0[16], a1[16];
        tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * 2) * ACC_W + (uint32_t)(t * 16), a0);
        tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * 2 + 1) * ACC_W + (uint32_t)(t * 16), a1);
        tmem_ld_wait();
#pragma unroll
        for (int n = 0; n < 16; ++n) y[n] = fmaf(__uint_as_float(a0[n]) + __uint_as_float(a1[n]), tw[t], y[n]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
      if (m < p.M) {
#pragma unroll
        for (int n = 0; n < 16; ++n) {
          if (n < p.N) {
            const float v = y[n] * g0r[n] * rsc;
            if (p.out_f32) reinterpret_cast<float*>(p.out)[(size_t)n * p.ldo + m] = v;
            else reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)n * p.ldo + m] = __float2bfloat16_rn(v);
          }
        }
      }
    }
  }
  __syncwarp();
  if (*abort_flag && threadIdx.x == 0) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) trace(4 * 16 + 2);
  if (warp == 2) tmem_dealloc(tmem_base, P_TMEM_COLS);
}

// ------------------------------------------------------------------ host
bool persist_on() {
  static const bool on = [] { const char* e = getenv("VELO_NO_PERSISTENT_GEMM"); return !(e && e[0] == '1'); }();
  return on;
}
int sm_count() {
  static const int n = [] {
    int dev = 0, v = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    return v > 0 ? v : 1;
  }();
  return n;
}
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode4() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(f);
  });
  return fn;
}
std::map<std::tuple<const void*, int>, CUtensorMap> g_bmaps;
std::mutex g_bmu;

int get_tmap_b(const void* bq, int ldb, int rows, CUtensorMap* out) {
  std::lock_guard<std::mutex> lk(g_bmu);
  auto key = std::make_tuple(bq, ldb * 4096 + rows / NT);
  auto it = g_bmaps.find(key);
  if (it != g_bmaps.end()) { *out = it->second; return 0; }
  EncodeTiledFn enc = get_encode4();
  if (!enc) return -1;
  cuuint64_t gdim[2] = {(cuuint64_t)ldb, (cuuint64_t)rows};
  cuuint64_t gstride[1] = {(cuuint64_t)ldb};
  cuuint32_t box[2] = {128, (cuuint32_t)NT};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap tm;
  CUresult r = enc(&tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(bq), gdim, gstride, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -(int)r - 100;
  if (g_bmaps.size() > 1024) g_bmaps.clear();
  g_bmaps[key] = tm;
  *out = tm;
  return 0;
}
}  // namespace

extern "C" int vg_gemm_fp4(const void* wt, const float* row_scale, const void* bq, int ldb, const void* sfb, const float* g0,
                           void* out, int out_f32, int M, int K, int N, int ldo, int splitk, int* err,
                           const VgCommCtx* ar_ctx, int ar_push_only, const VgConvEpi* conv, cudaStream_t stream) {
  if (M <= 0 || K <= 0 || N < 1 || N > 16 || splitk < 1 || splitk > 8 || (ldb % 128) != 0) return -2;
  Fp4Params p{};                  // every mode switch defaults to off
  p.wt = static_cast<const uint8_t*>(wt);
  p.row_scale = row_scale;
  p.sfb = static_cast<const uint8_t*>(sfb);
  p.g0 = g0;
  p.out = out;
  p.M = M; p.N = N; p.ldo = ldo;
  p.ks_total = (K + BKQ - 1) / BKQ;
  if (p.ks_total * (BKQ / 2) > ldb) return -4;
  p.out_f32 = out_f32;
  p.err = err;
  p.ar = 0;
  p.grouped = 0; p.tiles_per_expert = 0; p.x_div = 1; p.g_exp = nullptr; p.g_off = nullptr;
  p.has_conv = 0;
  if (conv && conv->conv_dim > 0) {
    if (conv->ck < 1 || conv->ck > CONV_MAX_CK || out_f32 || (ar_ctx && ar_ctx->world > 1)) return -6;
    p.has_conv = 1;
    p.conv = *conv;
  }
  if (ar_ctx && ar_ctx->world > 1) {
    if ((M + BM - 1) / BM > MAX_CTAS || (unsigned long long)N * M * 8ull > ar_ctx->slot_bytes) return -5;
    if (ar_push_only == 2 && (!ar_ctx->mc || (unsigned long long)N * M * 4ull > ar_ctx->mm_slot_bytes)) return -5;
    p.ar = ar_push_only == 2 ? 3 : (ar_push_only ? 2 : 1);
    p.comm = *ar_ctx;
  }
  if (splitk > p.ks_total) splitk = p.ks_total;
  CUtensorMap tm;
  int rc = get_tmap_b(bq, ldb, NT, &tm);
  if (rc) return rc;
  const int tiles = (M + BM - 1) / BM;
  if (splitk == 1 && !p.ar && !p.has_conv && p.ks_total >= 2 && tiles > sm_count() && persist_on()) {
    static bool configured_p = false;
    if (!configured_p) {
      cudaError_t e = cudaFuncSetAttribute(gemm_fp4_persist_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM_TOTAL);
      if (e != cudaSuccess) return (int)e;
      configured_p = true;
    }
    // Deep tile loops only (LM head): measured inside the decode chain, a persistent gate_up (1.8 tiles per SM)
    // is faster in isolation but ends on every SM at once, which costs the following kernels more overlap than
    // the kernel itself gains.
    static const int pmin = [] { const char* e = getenv("VELO_PERSIST_MIN_TILES"); return e ? atoi(e) : 4 * sm_count(); }();
    if (tiles >= pmin)
      return (int)launch_pdl(gemm_fp4_persist_kernel, dim3(sm_count()), dim3(THREADS), P_SMEM_TOTAL, stream, p, tm, tiles);
  }
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_fp4_kernel<NS>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL + CONV_SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  // (Measured and rejected for 1 < tiles / SMs <= 2, the gate_up case: two CTAs per SM on the two-stage ring, so that
  // every tile is resident at once. The shallow rings lose more bandwidth than the second wave's ramp costs:
  // 173 -> 157 tok/s on the 27B shape.)
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((M + BM - 1) / BM, 1, splitk);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = SMEM_TOTAL + ((p.has_conv || splitk > 1) ? CONV_SMEM : 0);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = splitk;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_on() ? 2 : 1;
  return (int)cudaLaunchKernelEx(&cfg, gemm_fp4_kernel<NS>, p, tm);
}

// MoE decode: `n_items` work items, item g = (expert g_exp[g] or -1, pair g_off[g]); the pair reads activation
// row pair / x_div of the quantised series (rows grouped sixteen to a B tile, `b_rows` = 64 * tiles) and writes
// out[pair][0 .. M). wt holds the experts stacked ([E * M, K] in the FP4 tile layout, M a multiple of 128).
extern "C" int vg_gemm_fp4_grouped(const void* wt, const float* row_scale, const void* bq, int ldb, int b_rows, const void* sfb,
                                   const float* g0, void* out, int out_f32, int M, int K, int ldo, int n_items, const int* g_exp,
                                   const int* g_off, int x_div, int* err, cudaStream_t stream) {
  if (M <= 0 || (M % BM) != 0 || K <= 0 || n_items < 1 || x_div < 1 || (ldb % 128) != 0 || (b_rows % NT) != 0) return -2;
  Fp4Params p{};                  // every mode switch defaults to off
  p.wt = static_cast<const uint8_t*>(wt);
  p.row_scale = row_scale;
  p.sfb = static_cast<const uint8_t*>(sfb);
  p.g0 = g0;
  p.out = out;
  p.M = M; p.N = 16; p.ldo = ldo;
  p.ks_total = (K + BKQ - 1) / BKQ;
  if (p.ks_total * (BKQ / 2) > ldb) return -4;
  p.out_f32 = out_f32;
  p.err = err;
  p.ar = 0;
  p.has_conv = 0;
  p.grouped = 1; p.tiles_per_expert = M / BM; p.x_div = x_div; p.g_exp = g_exp; p.g_off = g_off;
  CUtensorMap tm;
  int rc = get_tmap_b(bq, ldb, b_rows, &tm);
  if (rc) return rc;
  // Few work items (a single stream): the deep ring, one CTA per SM, as for the dense layers. Many items (wide
  // batches: hundreds of short K loops): the two-stage ring so that two CTAs share an SM.
  constexpr int GNS = 2;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_fp4_kernel<GNS>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_total(GNS));
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(gemm_fp4_kernel<NS>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL + CONV_SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  if ((long long)(M / BM) * n_items > 2ll * sm_count())
    return (int)launch_pdl(gemm_fp4_kernel<GNS>, dim3(M / BM, n_items, 1), dim3(THREADS), smem_total(GNS), stream, p, tm);
  return (int)launch_pdl(gemm_fp4_kernel<NS>, dim3(M / BM, n_items, 1), dim3(THREADS), SMEM_TOTAL, stream, p, tm);
}

VG_TRACE_SETTER(vg_trace_set_gemm_fp4)

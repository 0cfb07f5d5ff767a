// Weight-only quantized GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a.
//
//   Y[n, m] = row_scale[m] * sum_k dequant(W[m, k]) * X[n, k]
//
// "Swap-AB" orientation: the 128-row weight tile is the UMMA M operand, the activation columns are
// the UMMA N operand (16 for decode/verify, up to 128 for prefill), the fp32 accumulator lives in
// TMEM. One kernel covers every width, and for N <= 16 the instruction sequence, K order and split-K
// reduction order do not depend on N, so a column's bits are the same at width 1 and width 16.
// It takes the place of the reference's in-register-dequant mma.sync GEMM and of its
// dequantize-then-library-GEMM prefill path (reference: kernels/gpu_batch.cu:2846-2996,
// src/gpu.rs:2080-2185).
//
// Pipeline per CTA (384 threads = 12 warps; warp 11 idles):
//   warp 0      weight producer: 1-D bulk copies of pre-tiled packed weight slabs (128 rows x 128 k).
//   warp 10     activation producer: tiled tensor copies of the X slab (128-byte swizzle), no multicast.
//   warps 2-9   dequantizers: thread = weight row; e2m1 -> f16 with cvt, times the e4m3 block scale
//               (exact in f16), written with tcgen05.st straight into TMEM as the A operand, so the
//               expanded weights never touch shared memory. They also run the epilogue.
//   warp 1      allocates TMEM, issues tcgen05.mma (A from TMEM, B from shared memory; M=128, N=BN,
//               K=16) and commits to mbarriers.
// Unquantized (f16-tiled) weights skip the dequantizers: their tiles are bulk-copied into shared memory
// already in UMMA layout and used as a shared-memory A operand.
// Split-K runs as a thread-block cluster along z: partial tiles are summed through distributed
// shared memory in cluster-rank order by the rank-0 CTA, so no global scratch or atomics are needed.
// With a communication context the epilogue of a row-parallel GEMM is also the tensor-parallel all-reduce:
// fp32 partial tiles are pushed to all peers with plain stores over NVLink, a flag per (rank, tile) is
// raised with st.release.sys, and each rank adds the W partials in rank order - no separate collective.
// All mbarrier waits are bounded; on expiry an error code is stored to the status word and the CTA
// unwinds through its normal teardown (TMEM is always freed).
#include <cuda.h>
#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"
#include "api.h"

namespace {

using namespace vg;

constexpr int BM = 128;
constexpr int BK = 128;
constexpr int A_BYTES = BM * BK * 2;       // one f16 weight slab in shared memory (f16-tiled weights only)
constexpr int SUB_BYTES = BM * 128;        // one 64-wide K sub-tile of it
constexpr int A_COLS = BK / 2;             // TMEM columns of one dequantized slab (two f16 per column)
constexpr int NTHREADS = 384;

template <int WFMT> struct PackBytes;
template <> struct PackBytes<VG_WF_NVFP4> { static constexpr int v = 128 * 64 + 128 * 8; };
template <> struct PackBytes<VG_WF_FP8> { static constexpr int v = 128 * 128; };
template <> struct PackBytes<VG_WF_F16> { static constexpr int v = A_BYTES; };

struct GemmParams {
  const uint8_t* wt;
  const float* row_scale;
  void* out;
  int M, K, N, ldo;
  int ks_total;
  int out_f32;
  int* err;
#ifdef VG_TRACE      // profiling builds only
  int dbg;     // diagnostics: bit 0 skips the dequantisation math, bit 1 skips the MMA issue
  long long* trace;   // optional [9][64] cycle stamps of CTA (0,0,0): per-role pipeline events per slab
#endif
  // grouped (mixture-of-experts) mode: blockIdx.y walks work items = (group, n-tile)
  int grouped;
  const int* g_exp;      // [groups] expert of the group, -1 = not resident here (skipped)
  const int* g_off;      // [groups] first row of the group in X / Y
  const int* g_cnt;      // [groups] rows in the group
  const int* tilemap;    // [items][2] (group, n-tile) or null: item i = group i, n-tile 0
  const int* n_items;    // device count of valid items, or null: all of gridDim.y
  int tiles_per_expert;  // row tiles of one expert's matrix
  int x_div;             // X row = Y row / x_div (decode: one activation row feeds top-k pairs)
  // fused tensor-parallel reduction (row-parallel layers, N <= 16): the epilogue pushes this rank's fp32
  // partial tile into every rank's receive slot, raises a per-tile flag, waits for the other ranks' tiles
  // and stores the rank-order sum. ar == 0: plain store.
  int ar;
  int ag;                // 1: X is the all-gather landing zone; a token tile is loaded once its epoch word has arrived
  int ag_cap_rows;       // rows of one of the two landing-zone halves (the half is picked by the epoch's parity)
  int rs_rows;           // > 0: fused reduce-scatter epilogue, token rows [r * rs_rows, (r + 1) * rs_rows) belong to rank r
  VgCommCtx comm;
};

constexpr uint32_t pow2_cols(uint32_t c) { return c <= 32 ? 32 : c <= 64 ? 64 : c <= 128 ? 128 : c <= 256 ? 256 : 512; }

// NP: weight stages in shared memory; NA: slabs in flight between dequantizers / activation producer and
// the MMA issuers (TMEM A buffers and activation stages are released together by one commit).
template <int WFMT, int BN, int NP, int NA>
struct Cfg {
  static constexpr bool quant = WFMT != VG_WF_F16;
  static constexpr int pack = PackBytes<WFMT>::v;
  static constexpr int b_bytes = BN * BK * 2;
  static constexpr int b_off = 0;
  static constexpr int p_off = b_off + NA * b_bytes;              // multiple of 1024 for every BN >= 8
  static constexpr int bar_off = p_off + NP * pack;
  static constexpr int n_bars = 2 * NP + 3 * NA + 1;
  static constexpr int smem_total = bar_off + n_bars * 8 + 16 + 1024;
  static constexpr bool dual = BN <= 128;                          // two accumulators, one per MMA issuer
  static constexpr uint32_t acc_w = BN;                            // columns of one accumulator
  static constexpr uint32_t acc_cols = dual ? (2 * BN < 32 ? 32 : 2 * BN) : BN;
  static constexpr uint32_t tmem_cols = pow2_cols(acc_cols + (quant ? NA * A_COLS : 0));
  static_assert(NP * pack >= BN * BM * 4 || BN > 64, "split-K staging must fit in the weight stages");
  static_assert(NP % 2 == 0 && NA % 2 == 0, "ring sizes must be even: one MMA issuer per stage");
};

__device__ __forceinline__ uint32_t cvt_e4m3x2_f16x2(uint16_t v) {
  uint32_t r;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(v));
  return r;
}

// 8 e2m1 codes (one 32-bit word, low nibble first) times a block scale -> 8 f16 in 4 registers.
__device__ __forceinline__ void dequant8_fp4(uint32_t w, __half2 s2, uint32_t* o) {
  uint32_t h0, h1, h2, h3;
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
      "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t}\n"
      : "=r"(h0), "=r"(h1), "=r"(h2), "=r"(h3)
      : "r"(w));
  __half2 a = __hmul2(*reinterpret_cast<__half2*>(&h0), s2);
  __half2 b = __hmul2(*reinterpret_cast<__half2*>(&h1), s2);
  __half2 c = __hmul2(*reinterpret_cast<__half2*>(&h2), s2);
  __half2 d = __hmul2(*reinterpret_cast<__half2*>(&h3), s2);
  o[0] = *reinterpret_cast<uint32_t*>(&a);
  o[1] = *reinterpret_cast<uint32_t*>(&b);
  o[2] = *reinterpret_cast<uint32_t*>(&c);
  o[3] = *reinterpret_cast<uint32_t*>(&d);
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
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// A operand from TMEM, B operand from shared memory.
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

enum { TR_PROD = 0, TR_PACK_FULL, TR_MATH, TR_A_EMPTY, TR_ST_DONE, TR_MMA_A, TR_MMA_B, TR_MMA_DONE, TR_BPROD };
#ifdef VG_TRACE
__device__ __forceinline__ void stamp(const GemmParams& p, int role, int slab) {
  if (p.trace && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && slab < 64) p.trace[role * 64 + slab] = clock64();
}
#define VG_DBG(p, bit) ((p).dbg & (bit))
#else
__device__ __forceinline__ void stamp(const GemmParams&, int, int) {}
#define VG_DBG(p, bit) 0
#endif

__device__ __forceinline__ void report(int* err, int code, volatile int* abort_flag) {
  if (err) atomicCAS(err, 0, code);
  *abort_flag = 1;
}

template <int WFMT, int BN, int NP, int NA>
__global__ void __launch_bounds__(NTHREADS, 1)
gemm_tc_kernel(const GemmParams p, const __grid_constant__ CUtensorMap tmap_x) {
  using C = Cfg<WFMT, BN, NP, NA>;
  constexpr int PACK = C::pack;
  constexpr bool QUANT = C::quant;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sB = smem + C::b_off;
  uint8_t* sP = smem + C::p_off;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::bar_off);
  uint64_t* pack_full = bars;
  uint64_t* pack_empty = pack_full + NP;
  uint64_t* a_full = pack_empty + NP;       // dequantized slab is in TMEM
  uint64_t* b_full = a_full + NA;           // activation slab is in shared memory
  uint64_t* ab_empty = b_full + NA;         // the MMAs that read both have completed
  uint64_t* acc_full = ab_empty + NA;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  // successors launched with programmatic stream serialization may be scheduled once every CTA is here
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int mt = blockIdx.x, nt = blockIdx.y;
  const int S = gridDim.z, z = blockIdx.z;
  int row0 = nt * BN;              // first output row (token) of this CTA
  int rows_valid = p.N - row0;     // rows of it that exist
  int m_base = 0;                  // row offset of the expert inside the stacked weight
  if (p.grouped) {
    // uniform for the CTA (and its cluster): safe to leave before any barrier is touched
    if (p.n_items && (int)blockIdx.y >= *p.n_items) return;
    const int g = p.tilemap ? p.tilemap[2 * blockIdx.y] : (int)blockIdx.y;
    const int gnt = p.tilemap ? p.tilemap[2 * blockIdx.y + 1] : 0;
    const int e = p.g_exp[g];
    if (e < 0 || gnt * BN >= p.g_cnt[g]) return;
    row0 = p.g_off[g] + gnt * BN;
    rows_valid = p.g_cnt[g] - gnt * BN;
    mt = e * p.tiles_per_expert + (int)blockIdx.x;
    m_base = e * p.M;
    nt = 0;
  }
  const int x_row0 = p.grouped ? row0 / p.x_div : row0;
  // every CTA reads the collective epoch before any tile can publish the next one
  const uint32_t ar_epoch = (p.ar || p.rs_rows > 0 || p.ag) ? *p.comm.epoch + 1 : 0;
  const int ks0 = (int)(((long long)z * p.ks_total) / S);
  const int ks1 = (int)(((long long)(z + 1) * p.ks_total) / S);
  const int nks = ks1 - ks0;
  // Each row tile walks its K range from a different starting slab (wrapping around), so the CTAs of a
  // wave do not all ask L2 for the same activation lines at the same moment. The order is a function of
  // the tile index only, hence identical for every batch width.
  const int rot = nks > 0 ? (int)(((unsigned)blockIdx.x * 7u + (unsigned)z * 3u) % (unsigned)nks) : 0;
  auto slab_of = [&](int i) { int k = i + rot; return ks0 + (k >= nks ? k - nks : k); };

  if (threadIdx.x == 0) {
    // quantized: pack_empty is released by the 8 dequantizer warps; f16 tiles: by the MMA commit
    for (int i = 0; i < NP; ++i) { mbar_init(&pack_full[i], 1); mbar_init(&pack_empty[i], QUANT ? 8 : 1); }
    for (int i = 0; i < NA; ++i) { mbar_init(&a_full[i], 8); mbar_init(&b_full[i], 1); mbar_init(&ab_empty[i], 1); }
    mbar_init(acc_full, C::dual ? 2 : 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_a0 = tmem_base + C::acc_cols;

  if (warp == 0) {
    // ------------------------------------------------ weight producer
    if (lane == 0) {
      for (int i = 0; i < nks && !*abort_flag; ++i) {
        const int s = i % NP;
        if (!mbar_wait(&pack_empty[s], ((i / NP) & 1) ^ 1)) { report(p.err, VG_ERR_EMPTY_WAIT, abort_flag); break; }
        stamp(p, TR_PROD, i);
        mbar_arrive_expect_tx(&pack_full[s], PACK);
        tma_bulk_g2s(sP + (size_t)s * PACK, p.wt + ((size_t)mt * p.ks_total + slab_of(i)) * PACK, PACK, &pack_full[s]);
      }
    }
  } else if (warp == 10) {
    // ------------------------------------------------ activation producer
    if (lane == 0) {
      if (p.ag) {
        // fused all-gather: the 128-row tiles this CTA reads must have landed (pushed by their owner rank)
        const uint32_t* fl = reinterpret_cast<const uint32_t*>(p.comm.data[p.comm.rank] + p.comm.agflags_off) +
                             (size_t)(ar_epoch & 1) * VG_AG_MAX_TILES;
        const int t_lo = x_row0 / 128, t_hi = (min(x_row0 + BN, p.N) - 1) / 128;
        for (int t = t_lo; t <= t_hi; ++t)
          if (!wait_flag(fl + t, ar_epoch, p.comm.timeout_ns)) { atomicCAS(p.comm.status, 0, VG_ERR_PEER_WAIT); *abort_flag = 1; }
        asm volatile("fence.proxy.async;" ::: "memory");    // the rows were written through the generic proxy
      }
      const int x_row = x_row0 + (p.ag ? (int)(ar_epoch & 1) * p.ag_cap_rows : 0);
      for (int i = 0; i < nks && !*abort_flag; ++i) {
        const int b = i % NA;
        if (!mbar_wait(&ab_empty[b], ((i / NA) & 1) ^ 1)) { report(p.err, VG_ERR_EMPTY_WAIT, abort_flag); break; }
        stamp(p, TR_BPROD, i);
        mbar_arrive_expect_tx(&b_full[b], C::b_bytes);
        uint8_t* bdst = sB + (size_t)b * C::b_bytes;
        const int ks = slab_of(i);
        tma_tensor2d_g2s(bdst, &tmap_x, ks * BK, x_row, &b_full[b]);
        tma_tensor2d_g2s(bdst + BN * 128, &tmap_x, ks * BK + 64, x_row, &b_full[b]);
      }
    }
  } else if (warp == 1 || warp == 11) {
    // ------------------------------------------------ MMA issuers: even slabs -> accumulator 0 (warp 1),
    // odd slabs -> accumulator 1 (warp 11). The epilogue adds the two in a fixed order. The 256-token tile has
    // one accumulator (it fills half of TMEM by itself) and one issuer.
    constexpr int STEP = C::dual ? 2 : 1;
    if (lane == 0 && (C::dual || warp == 1)) {
      constexpr uint32_t idesc = umma_idesc_f16(BM, BN, 0, 0);
      const int me = warp == 1 ? 0 : 1;
      const uint32_t tmem_acc = tmem_base + (uint32_t)me * C::acc_w;
      bool ok = true;
      for (int i = me; i < nks && !*abort_flag; i += STEP) {
        const int a = i % NA;
        const int sp = i % NP;
        if (QUANT) {
          if (!mbar_wait(&a_full[a], (i / NA) & 1)) { report(p.err, VG_ERR_DEQ_WAIT, abort_flag); ok = false; break; }
        } else {
          if (!mbar_wait(&pack_full[sp], (i / NP) & 1)) { report(p.err, VG_ERR_TMA_WAIT, abort_flag); ok = false; break; }
        }
        stamp(p, TR_MMA_A, i);
        if (!mbar_wait(&b_full[a], (i / NA) & 1)) { report(p.err, VG_ERR_TMA_WAIT, abort_flag); ok = false; break; }
        stamp(p, TR_MMA_B, i);
        tc_fence_after();
        const uint32_t b_addr = smem_u32(sB + (size_t)a * C::b_bytes);
        if (!VG_DBG(p, 2)) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint64_t bd = umma_desc_sw128(b_addr + (kk >> 2) * (BN * 128) + (kk & 3) * 32);
            const uint32_t acc_flag = (i >= STEP || kk != 0) ? 1u : 0u;
            if (QUANT) {
              umma_f16_ts(tmem_acc, tmem_a0 + (uint32_t)(a * A_COLS + kk * 8), bd, idesc, acc_flag);
            } else {
              const uint32_t a_addr = smem_u32(sP + (size_t)sp * PACK);
              umma_f16(tmem_acc, umma_desc_sw128(a_addr + (kk >> 2) * SUB_BYTES + (kk & 3) * 32), bd, idesc, acc_flag);
            }
          }
        }
        umma_commit(&ab_empty[a]);
        if (!QUANT) umma_commit(&pack_empty[sp]);
        stamp(p, TR_MMA_DONE, i);
      }
      if (ok) umma_commit(acc_full);
    }
  } else if (QUANT) {
    // ------------------------------------------------ dequantizers (warps 2..9): thread = weight row
    const int q = warp & 3;                      // TMEM lane quarter this warp owns
    const int half = (warp - 2) >> 2;            // which 64-wide half of the slab's K range
    const int r = q * 32 + lane;
    const int rs = r & 7;
    for (int i = 0; i < nks && !*abort_flag; ++i) {
      const int s = i % NP, a = i % NA;
      if (!mbar_wait(&pack_full[s], (i / NP) & 1)) { report(p.err, VG_ERR_TMA_WAIT, abort_flag); break; }
      if (warp == 2 && lane == 0) stamp(p, TR_PACK_FULL, i);
      const uint8_t* pk = sP + (size_t)s * PACK;
      uint32_t v[32];
      if (VG_DBG(p, 1)) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = 0;
      } else if (WFMT == VG_WF_NVFP4) {
        const int sw = (r >> 1) & 3;
        const uint4 p0 = *reinterpret_cast<const uint4*>(pk + r * 64 + (((2 * half) ^ sw) << 4));
        const uint4 p1 = *reinterpret_cast<const uint4*>(pk + r * 64 + (((2 * half + 1) ^ sw) << 4));
        const uint32_t sc = *reinterpret_cast<const uint32_t*>(pk + 8192 + r * 8 + half * 4);
        uint32_t s01 = cvt_e4m3x2_f16x2((uint16_t)(sc & 0xffff));
        uint32_t s23 = cvt_e4m3x2_f16x2((uint16_t)(sc >> 16));
        const __half2 h01 = *reinterpret_cast<__half2*>(&s01);
        const __half2 h23 = *reinterpret_cast<__half2*>(&s23);
        const __half2 sc0 = __low2half2(h01), sc1 = __high2half2(h01);
        const __half2 sc2 = __low2half2(h23), sc3 = __high2half2(h23);
        dequant8_fp4(p0.x, sc0, v + 0);  dequant8_fp4(p0.y, sc0, v + 4);
        dequant8_fp4(p0.z, sc1, v + 8);  dequant8_fp4(p0.w, sc1, v + 12);
        dequant8_fp4(p1.x, sc2, v + 16); dequant8_fp4(p1.y, sc2, v + 20);
        dequant8_fp4(p1.z, sc3, v + 24); dequant8_fp4(p1.w, sc3, v + 28);
      } else {
        // FP8: row r holds 128 code bytes in eight 16-byte chunks stored at chunk ^ (r & 7).
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint4 qv = *reinterpret_cast<const uint4*>(pk + r * 128 + (((half * 4 + c) ^ rs) << 4));
          v[c * 8 + 0] = cvt_e4m3x2_f16x2((uint16_t)(qv.x & 0xffff)); v[c * 8 + 1] = cvt_e4m3x2_f16x2((uint16_t)(qv.x >> 16));
          v[c * 8 + 2] = cvt_e4m3x2_f16x2((uint16_t)(qv.y & 0xffff)); v[c * 8 + 3] = cvt_e4m3x2_f16x2((uint16_t)(qv.y >> 16));
          v[c * 8 + 4] = cvt_e4m3x2_f16x2((uint16_t)(qv.z & 0xffff)); v[c * 8 + 5] = cvt_e4m3x2_f16x2((uint16_t)(qv.z >> 16));
          v[c * 8 + 6] = cvt_e4m3x2_f16x2((uint16_t)(qv.w & 0xffff)); v[c * 8 + 7] = cvt_e4m3x2_f16x2((uint16_t)(qv.w >> 16));
        }
      }
      // the packed stage is consumed: hand it back before waiting for a free TMEM slab
      __syncwarp();
      if (warp == 2 && lane == 0) stamp(p, TR_MATH, i);
      if (lane == 0) mbar_arrive(&pack_empty[s]);
      if (!mbar_wait(&ab_empty[a], ((i / NA) & 1) ^ 1)) { report(p.err, VG_ERR_EMPTY_WAIT, abort_flag); break; }
      if (warp == 2 && lane == 0) stamp(p, TR_A_EMPTY, i);
      tc_fence_after();
      tmem_st32(tmem_a0 + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * A_COLS + half * 32), v);
      tmem_st_wait();
      if (warp == 2 && lane == 0) stamp(p, TR_ST_DONE, i);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&a_full[a]);
    }
  }
  __syncwarp();

  // ---------------------------------------------------- epilogue (warps 2..9)
  // A pass covers 2 x CPW token columns (the two warp groups side by side); only the 256-token tile, which
  // has neither split-K nor a fused reduction, takes two passes.
  constexpr int CPW = BN >= 256 ? 64 : BN / 2;   // accumulator columns handled by one warp in one pass
  constexpr int PASSES = BN / (2 * CPW);
  const int q = warp & 3;                // TMEM lane quarter this warp may read
  const int grp = warp >= 6 ? 1 : 0;     // which half of the pass's columns
  const int m_local = q * 32 + lane;
  const bool epi = warp >= 2 && warp <= 9;
  for (int ps = 0; ps < PASSES; ++ps) {
  const int cb = ps * 2 * CPW + grp * CPW;       // first token column of this warp in this pass
  float acc[CPW];
  bool have_acc = false;
  if (epi) {
    if (mbar_wait(acc_full, 0)) {
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < CPW; c += 8) {
        uint32_t v0[8], v1[8];
        tmem_ld8(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(cb + c), v0);
        if (C::dual) tmem_ld8(tmem_base + ((uint32_t)(q * 32) << 16) + C::acc_w + (uint32_t)(cb + c), v1);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 8; ++j)
          acc[c + j] = (C::dual && nks >= 2) ? __uint_as_float(v0[j]) + __uint_as_float(v1[j]) : __uint_as_float(v0[j]);
      }
      have_acc = true;
    } else {
      report(p.err, VG_ERR_MMA_WAIT, abort_flag);
    }
  }
  if (S > 1) {
    // Partial tiles go through distributed shared memory; cluster rank 0 sums them in rank order.
    // The weight stages are idle by now (every MMA has completed) and serve as the staging buffer.
    float* red = reinterpret_cast<float*>(sP);
    if (epi && have_acc) {
#pragma unroll
      for (int c = 0; c < CPW; ++c) red[(cb + c) * BM + m_local] = acc[c];
    }
    cluster_sync_all();
    if (z == 0 && epi && have_acc) {
      const uint32_t red_addr = smem_u32(red);
      for (int s = 1; s < S; ++s) {
        const uint32_t remote = dsmem_map(red_addr, (uint32_t)s);
#pragma unroll
        for (int c = 0; c < CPW; ++c) acc[c] += dsmem_ld_f32(remote + (uint32_t)(((cb + c) * BM + m_local) * 4));
      }
    }
    cluster_sync_all();
  }
  if (epi && z == 0 && p.ar) {
    // ---- fused all-reduce epilogue (all 256 epilogue threads take part, also on the error path)
    __shared__ int ar_failed;
    const VgCommCtx& c = p.comm;
    const uint32_t e = ar_epoch;
    const int set = e & 1;
    const int et = threadIdx.x - 64;                      // 0..255 among the epilogue warps
    const int m = (int)blockIdx.x * BM + m_local;
    const float rsc = (p.row_scale && m < p.M) ? p.row_scale[m] : 1.0f;
    if (et == 0) ar_failed = 0;
    if (have_acc && m < p.M) {
      for (int k = 0; k < c.world; ++k) {
        const int peer = (c.rank + k) % c.world;
        float* dst = reinterpret_cast<float*>(c.data[peer] + c.slots_off + (size_t)(set * MAX_RANKS + c.rank) * c.slot_bytes);
#pragma unroll
        for (int cc = 0; cc < CPW; ++cc) {
          const int col = cb + cc;
          if (col < rows_valid) dst[(size_t)(row0 + col) * p.M + m] = acc[cc] * rsc;
        }
      }
    }
    __threadfence_system();
    asm volatile("bar.sync 1, 256;" ::: "memory");
    if (et < c.world)
      st_release_sys(reinterpret_cast<uint32_t*>(c.data[et] + c.flags_off) + flag_index(set, c.rank, (int)blockIdx.x), e);
    if (et < c.world) {
      const uint32_t* f = reinterpret_cast<const uint32_t*>(c.data[c.rank] + c.flags_off) + flag_index(set, et, (int)blockIdx.x);
      if (!wait_flag(f, e, c.timeout_ns)) { atomicCAS(c.status, 0, VG_ERR_PEER_WAIT); ar_failed = 1; }
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");
    if (!ar_failed && have_acc && m < p.M) {
      const float* base = reinterpret_cast<const float*>(c.data[c.rank] + c.slots_off + (size_t)set * MAX_RANKS * c.slot_bytes);
      const size_t stride = c.slot_bytes / sizeof(float);
#pragma unroll
      for (int cc = 0; cc < CPW; ++cc) {
        const int col = cb + cc;
        if (col < rows_valid) {
          const size_t idx = (size_t)(row0 + col) * p.M + m;
          float sum = 0.f;
          for (int q2 = 0; q2 < c.world; ++q2) sum += __ldcg(&base[(size_t)q2 * stride + idx]);
          if (p.out_f32) reinterpret_cast<float*>(p.out)[(size_t)(row0 + col) * p.ldo + m] = sum;
          else reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)(row0 + col) * p.ldo + m] = __float2bfloat16_rn(sum);
        }
      }
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");
    if (et == 0) {
      // the last tile to finish publishes the new epoch for the next collective
      __threadfence();
      if (atomicAdd(c.done_ctr, 1u) == gridDim.x * gridDim.y - 1) { *c.done_ctr = 0; *c.epoch = e; }
    }
  } else if (epi && z == 0 && p.rs_rows > 0) {
    // ---- fused reduce-scatter: this tile's token rows belong to one rank; its fp32 partial goes straight into
    // that rank's receive slot over NVLink, then the tile's epoch is published there. No waiting here: the sum and
    // the all-gather run in vg_comm_gemm_rs_finish while later tiles of this GEMM are still computing.
    const VgCommCtx& c = p.comm;
    const uint32_t e = ar_epoch;
    const int set = e & 1;
    const int et = threadIdx.x - 64;
    const int m = (int)blockIdx.x * BM + m_local;
    const int owner = row0 / p.rs_rows;
    const int lrow0 = row0 - owner * p.rs_rows;
    const float rsc = (p.row_scale && m < p.M) ? p.row_scale[m] : 1.0f;
    if (have_acc && m < p.M) {
      float* dst = reinterpret_cast<float*>(c.data[owner] + c.slots_off + (size_t)(set * MAX_RANKS + c.rank) * c.slot_bytes);
#pragma unroll
      for (int cc = 0; cc < CPW; ++cc) {
        const int col = cb + cc;
        if (col < rows_valid) dst[(size_t)(lrow0 + col) * p.M + m] = acc[cc] * rsc;
      }
    }
    __threadfence_system();
    asm volatile("bar.sync 1, 256;" ::: "memory");
    if (et == 0) {
      // flags are per 128 token rows: a 256-token tile publishes one word per pass
      const int tile = ((lrow0 + ps * 2 * CPW) / 128) * (int)gridDim.x + (int)blockIdx.x;
      st_release_sys(reinterpret_cast<uint32_t*>(c.data[owner] + c.rsflags_off) +
                         ((size_t)(set * MAX_RANKS + c.rank) * VG_RS_MAX_TILES + tile), e);
    }
  } else if (epi && have_acc && z == 0) {
    const int m = (int)blockIdx.x * BM + m_local;       // row inside this (expert's) matrix
    if (m < p.M) {
      const float rsc = p.row_scale ? p.row_scale[m_base + m] : 1.0f;
#pragma unroll
      for (int c = 0; c < CPW; ++c) {
        const int cc = cb + c;
        const int n = row0 + cc;
        if (cc < rows_valid) {
          const float v = acc[c] * rsc;
          if (p.out_f32) reinterpret_cast<float*>(p.out)[(size_t)n * p.ldo + m] = v;
          else reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)n * p.ldo + m] = __float2bfloat16_rn(v);
        }
      }
    }
  }
  }  // passes
  if (p.ag && threadIdx.x == 64) {
    // the last CTA to finish publishes the epoch: the landing zone may be overwritten by the next gather
    __threadfence();
    if (atomicAdd(p.comm.done_ctr, 1u) == gridDim.x * gridDim.y * gridDim.z - 1) { *p.comm.done_ctr = 0; *p.comm.epoch = ar_epoch; }
  }
  if (*abort_flag && threadIdx.x == 0) {
    // Give bulk copies that may still be in flight time to land before shared memory is released.
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, C::tmem_cols);
}

// ------------------------------------------------------------------ host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
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

struct TmapKey {
  const void* ptr; int rows, k, bn, ldx;
  bool operator<(const TmapKey& o) const {
    return std::tie(ptr, rows, k, bn, ldx) < std::tie(o.ptr, o.rows, o.k, o.bn, o.ldx);
  }
};
#ifdef VG_TRACE
int g_dbg = 0;
long long* g_trace = nullptr;
#endif
std::map<TmapKey, CUtensorMap> g_tmaps;
std::mutex g_tmap_mu;

// Tensor map over X [rows, K] f16, row stride ldx elements; box = 64 k-elements x BN rows, 128-byte
// swizzle. Rows beyond `rows` and k beyond K are zero-filled by the copy engine without touching memory.
int get_tmap_x(const void* x, int rows, int K, int bn, int ldx, CUtensorMap* out) {
  std::lock_guard<std::mutex> lk(g_tmap_mu);
  TmapKey key{x, rows, K, bn, ldx};
  auto it = g_tmaps.find(key);
  if (it != g_tmaps.end()) { *out = it->second; return 0; }
  EncodeTiledFn enc = get_encode();
  if (!enc) return -1;
  cuuint64_t gdim[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t gstride[1] = {(cuuint64_t)ldx * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)bn};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap tm;
  CUresult r = enc(&tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(x), gdim, gstride, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -(int)r - 100;
  if (g_tmaps.size() > 4096) g_tmaps.clear();
  g_tmaps[key] = tm;
  *out = tm;
  return 0;
}

template <int WFMT, int BN, int NP, int NA>
int launch(const GemmParams& p, const CUtensorMap& tm, int splitk, cudaStream_t st) {
  using C = Cfg<WFMT, BN, NP, NA>;
  auto kern = gemm_tc_kernel<WFMT, BN, NP, NA>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::smem_total);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((p.M + BM - 1) / BM, (p.N + BN - 1) / BN, splitk);
  cfg.blockDim = dim3(NTHREADS);
  cfg.dynamicSmemBytes = C::smem_total;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = splitk;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  // Launched as an ordinary dependent (measured: starting this kernel's CTAs early only takes SM slots from the
  // kernel it waits for); the trigger at its top still lets its own successor be scheduled early.
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, kern, p, tm);
}

// Stage counts. Both ring sizes are even: slab i always lands in a stage of the same parity as i, so each
// stage and each of its barriers is consumed by one MMA issuer only, in order. (With an odd ring an
// issuer would skip every other phase of a barrier and a one-bit parity wait could pass a phase early
// when bulk copies complete out of order.) NVFP4 decode keeps 8 x 9 KB weight stages in flight per CTA
// and fits two CTAs per SM.
template <int WFMT, int BN> struct Stages;
template <int BN> struct Stages<VG_WF_NVFP4, BN> { static constexpr int np = BN <= 64 ? 8 : 6, na = 2; };
template <int BN> struct Stages<VG_WF_FP8, BN> { static constexpr int np = 4, na = 2; };
template <int BN> struct Stages<VG_WF_F16, BN> { static constexpr int np = BN >= 256 ? 2 : 4, na = 2; };

template <int WFMT, int BN>
int launch_bn(const GemmParams& p, const CUtensorMap& tm, int splitk, cudaStream_t st) {
  using S = Stages<WFMT, BN>;
  return launch<WFMT, BN, S::np, S::na>(p, tm, splitk, st);
}

bool wide_tiles_on() {
  static const bool on = [] { const char* e = getenv("VELO_NO_WIDE_TILES"); return !(e && e[0] == '1'); }();
  return on;
}
int sm_count_tc() {
  static const int n = [] { int dev = 0, sms = 148; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); return sms; }();
  return n;
}

template <int WFMT>
int dispatch_bn(const GemmParams& p, const void* x, int ldx, int splitk, cudaStream_t st) {
  CUtensorMap tm;
  int bn = p.N <= 16 ? 16 : (p.N <= 32 ? 32 : (p.N <= 64 ? 64 : 128));
  // 256-token tiles for wide prefill GEMMs: every dequantised weight slab feeds twice the MMA work, which hides
  // the dequantisers' latency (the 128-token tile leaves the tensor pipe idle more than half of the time). Only
  // when the grid still fills the GPU twice over, and with the fused reduce-scatter only when no tile straddles
  // two owners (its flags stay per 128 token rows).
  if (p.N > 128 && (p.rs_rows % 256) == 0 && wide_tiles_on() &&
      (long long)((p.M + BM - 1) / BM) * ((p.N + 255) / 256) >= 2ll * sm_count_tc())
    bn = 256;
  int rc = get_tmap_x(x, p.ag ? 2 * p.ag_cap_rows : p.N, p.K, bn, ldx, &tm);
  if (rc) return rc;
  switch (bn) {
    case 16: return launch_bn<WFMT, 16>(p, tm, splitk, st);
    case 32: return launch_bn<WFMT, 32>(p, tm, splitk, st);
    case 64: return launch_bn<WFMT, 64>(p, tm, splitk, st);
    case 256: return launch_bn<WFMT, 256>(p, tm, splitk, st);
    default: return launch_bn<WFMT, 128>(p, tm, splitk, st);
  }
}

}  // namespace

extern "C" int vg_gemm_tc(const void* wt, const float* row_scale, const void* x_f16, int x_rows, int ldx, void* out,
                          int out_f32, int M, int K, int N, int ldo, int wfmt, int splitk, int* err,
                          const VgCommCtx* ar_ctx, int rs_rows, int ag, cudaStream_t stream) {
  if (M <= 0 || K <= 0 || N <= 0 || (K % 16) != 0 || splitk < 1 || splitk > 8 || x_rows < N) return -2;
  if (ldx < K || (ldx % 8) != 0 || (reinterpret_cast<uintptr_t>(x_f16) & 15) != 0) return -4;
  GemmParams p{};                 // every mode switch defaults to off
  p.wt = static_cast<const uint8_t*>(wt);
  p.row_scale = row_scale;
  p.out = out;
  p.M = M; p.K = K; p.N = N; p.ldo = ldo;
  p.ks_total = (K + BK - 1) / BK;
  p.out_f32 = out_f32;
  p.err = err;
#ifdef VG_TRACE
  p.dbg = g_dbg;
  p.trace = g_trace;
#endif
  p.grouped = 0;
  p.ar = 0;
  p.rs_rows = 0;
  p.ag = 0;
  if (ar_ctx && ar_ctx->world > 1 && ag) {
    // fused all-gather: X must be this rank's landing zone, whole problem in one launch, plain epilogue
    const long long cap_rows = (long long)(ar_ctx->agbuf_bytes / 2 / ((unsigned long long)K * 2ull)) / 128 * 128;
    if (rs_rows > 0 || splitk != 1 || (N + 127) / 128 > VG_AG_MAX_TILES || ldx != K || N > cap_rows ||
        x_f16 != (const void*)(ar_ctx->data[ar_ctx->rank] + ar_ctx->agbuf_off) || x_rows != 2 * cap_rows)
      return -5;
    p.ag = 1;
    p.ag_cap_rows = (int)cap_rows;
    p.comm = *ar_ctx;
  } else if (ar_ctx && ar_ctx->world > 1 && rs_rows > 0) {
    // fused reduce-scatter (prefill widths): whole 128-token tiles per owner, every tile has a flag word
    const long long tiles = (long long)((rs_rows + 127) / 128) * ((M + BM - 1) / BM);
    if (N <= 64 || (rs_rows % 128) != 0 || out_f32 || tiles > VG_RS_MAX_TILES || splitk != 1 ||
        (unsigned long long)rs_rows * M * 4ull > ar_ctx->slot_bytes || (long long)rs_rows * ar_ctx->world < N)
      return -5;
    p.rs_rows = rs_rows;
    p.comm = *ar_ctx;
  } else if (ar_ctx && ar_ctx->world > 1) {
    // fused reduction: decode widths only, one flag per row tile
    if (N > 16 || (M + BM - 1) / BM > MAX_CTAS || (unsigned long long)N * M * 4ull > ar_ctx->slot_bytes) return -5;
    p.ar = 1;
    p.comm = *ar_ctx;
  }
  if (splitk > p.ks_total) splitk = p.ks_total;
  if (N > 64) splitk = 1;
  switch (wfmt) {
    case VG_WF_NVFP4: return dispatch_bn<VG_WF_NVFP4>(p, x_f16, ldx, splitk, stream);
    case VG_WF_FP8: return dispatch_bn<VG_WF_FP8>(p, x_f16, ldx, splitk, stream);
    case VG_WF_F16: return dispatch_bn<VG_WF_F16>(p, x_f16, ldx, splitk, stream);
  }
  return -3;
}

// Grouped (mixture-of-experts) GEMM over stacked expert weights [E][M, K] (tile-major per expert).
// Work item i (blockIdx.y) = (group, n-tile): rows [g_off[g] + nt*BN, ...) of X/Y use expert g_exp[g].
// bn selects the tile width: 16 for decode (one pair per group), 128 for prefill (tokens sorted by expert).
extern "C" int vg_gemm_tc_grouped(const void* wt, const float* row_scale, const void* x_f16, int x_rows, int ldx, void* out,
                                  int out_f32, int M, int K, int ldo, int wfmt, int bn, int max_items, const int* g_exp,
                                  const int* g_off, const int* g_cnt, const int* tilemap, const int* n_items, int x_div,
                                  int* err, cudaStream_t stream) {
  if (M <= 0 || K <= 0 || max_items <= 0 || (K % 16) != 0 || (M % BM) != 0 || x_div < 1) return -2;
  if (ldx < K || (ldx % 8) != 0 || (reinterpret_cast<uintptr_t>(x_f16) & 15) != 0) return -4;
  GemmParams p{};                 // every mode switch defaults to off
  p.wt = static_cast<const uint8_t*>(wt);
  p.row_scale = row_scale;
  p.out = out;
  p.M = M; p.K = K; p.ldo = ldo;
  p.N = bn == 16 ? 16 : 128;                 // selects the tile width; the real row counts come from g_cnt
  p.ks_total = (K + BK - 1) / BK;
  p.out_f32 = out_f32;
  p.err = err;
  p.grouped = 1;
  p.ar = 0;
  p.rs_rows = 0;
  p.g_exp = g_exp; p.g_off = g_off; p.g_cnt = g_cnt; p.tilemap = tilemap; p.n_items = n_items;
  p.tiles_per_expert = M / BM;
  p.x_div = x_div;
  CUtensorMap tm;
  int rc = get_tmap_x(x_f16, x_rows, K, bn == 16 ? 16 : 128, ldx, &tm);
  if (rc) return rc;
  // items ride on gridDim.y: launch() derives gridDim.y from N, so pass N = items * tile width
  GemmParams q = p;
  q.N = max_items * (bn == 16 ? 16 : 128);
  switch (wfmt) {
    case VG_WF_NVFP4: return bn == 16 ? launch_bn<VG_WF_NVFP4, 16>(q, tm, 1, stream) : launch_bn<VG_WF_NVFP4, 128>(q, tm, 1, stream);
    case VG_WF_FP8: return bn == 16 ? launch_bn<VG_WF_FP8, 16>(q, tm, 1, stream) : launch_bn<VG_WF_FP8, 128>(q, tm, 1, stream);
    case VG_WF_F16: return bn == 16 ? launch_bn<VG_WF_F16, 16>(q, tm, 1, stream) : launch_bn<VG_WF_F16, 128>(q, tm, 1, stream);
  }
  return -3;
}

// Profiling builds (-DVG_TRACE) only: diagnostic flags (see GemmParams::dbg) and a device buffer of 9 x 64 int64
// that receives cycle stamps of CTA (0,0,0)'s pipeline events (null = off). Returns -1 in a regular build.
extern "C" int vg_gemm_tc_set_debug(int dbg, long long* trace_buf) {
#ifdef VG_TRACE
  g_dbg = dbg;
  g_trace = trace_buf;
  return 0;
#else
  (void)dbg; (void)trace_buf;
  return -1;
#endif
}

// Number of CTAs of the decode configuration that can be resident at once (used by the host
// heuristic that picks the split-K factor).
extern "C" int vg_gemm_tc_resident_ctas(int wfmt) {
  int dev = 0, sms = 0, per_sm = 1;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // residency of the decode tile from its resources: shared memory (1 KB reserved per CTA, 228 KB per SM),
  // TMEM columns (512 per SM) and threads
  auto fit = [](int smem, unsigned cols) {
    int by_smem = (228 * 1024) / (smem + 1024);
    int by_tmem = (int)(512 / cols);
    int by_thr = 2048 / NTHREADS;
    int r = by_smem < by_tmem ? by_smem : by_tmem;
    return r < by_thr ? r : by_thr;
  };
  if (wfmt == VG_WF_NVFP4) {
    using S = Stages<VG_WF_NVFP4, 16>;
    using C = Cfg<VG_WF_NVFP4, 16, S::np, S::na>;
    per_sm = fit(C::smem_total, C::tmem_cols);
  } else if (wfmt == VG_WF_FP8) {
    using S = Stages<VG_WF_FP8, 16>;
    using C = Cfg<VG_WF_FP8, 16, S::np, S::na>;
    per_sm = fit(C::smem_total, C::tmem_cols);
  } else {
    using S = Stages<VG_WF_F16, 16>;
    using C = Cfg<VG_WF_F16, 16, S::np, S::na>;
    per_sm = fit(C::smem_total, C::tmem_cols);
  }
  return sms * (per_sm > 0 ? per_sm : 1);
}

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
// Pipeline per CTA (320 threads):
//   warp 0      TMA producer: 1-D bulk copies of pre-tiled packed weight slabs (128 rows x 128 k) and
//               tiled tensor copies of the activation slab (128-byte swizzle), no multicast.
//   warps 2-9   dequantize a packed slab from shared memory into an f16 K-major swizzled UMMA tile
//               (e2m1 -> f16 with cvt, times the e4m3 block scale; exact in f16), then run the epilogue.
//   warp 1      allocates TMEM, issues tcgen05.mma (M=128, N=BN, K=16) and commits to mbarriers.
// Split-K runs as a thread-block cluster along z: partial tiles are summed through distributed
// shared memory in cluster-rank order by the rank-0 CTA, so no global scratch or atomics are needed.
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
constexpr int A_BYTES = BM * BK * 2;       // one dequantized f16 weight slab
constexpr int SUB_BYTES = BM * 128;        // one 64-wide K sub-tile of it

template <int WFMT> struct PackBytes;
template <> struct PackBytes<VG_WF_NVFP4> { static constexpr int v = 128 * 64 + 128 * 8; };
template <> struct PackBytes<VG_WF_FP8> { static constexpr int v = 128 * 128; };
template <> struct PackBytes<VG_WF_F16> { static constexpr int v = 0; };

struct GemmParams {
  const uint8_t* wt;
  const float* row_scale;
  void* out;
  int M, K, N, ldo;
  int ks_total;
  int out_f32;
  int* err;
};

template <int WFMT, int BN, int NP, int NA, int NB>
struct SmemLayout {
  static constexpr int b_bytes = BN * BK * 2;
  static constexpr int a_off = 0;
  static constexpr int b_off = a_off + NA * A_BYTES;
  static constexpr int p_off = b_off + NB * b_bytes;
  static constexpr int bar_off = p_off + NP * PackBytes<WFMT>::v;
  static constexpr int n_bars = 2 * NP + 2 * NA + 2 * NB + 1;
  static constexpr int total = bar_off + n_bars * 8 + 16 + 1024;   // + tmem slot/abort + alignment slack
};

__device__ __forceinline__ uint32_t cvt_e4m3x2_f16x2(uint16_t v) {
  uint32_t r;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(v));
  return r;
}

// 8 e2m1 codes (one 32-bit word, low nibble first) times a block scale -> 8 f16 in a uint4.
__device__ __forceinline__ uint4 dequant8_fp4(uint32_t w, __half2 s2) {
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
  uint4 o;
  o.x = *reinterpret_cast<uint32_t*>(&a);
  o.y = *reinterpret_cast<uint32_t*>(&b);
  o.z = *reinterpret_cast<uint32_t*>(&c);
  o.w = *reinterpret_cast<uint32_t*>(&d);
  return o;
}

__device__ __forceinline__ void report(int* err, int code, volatile int* abort_flag) {
  if (err) atomicCAS(err, 0, code);
  *abort_flag = 1;
}

template <int WFMT, int BN, int NP_, int NA, int NB>
__global__ void __launch_bounds__(320, 1)
gemm_tc_kernel(const GemmParams p, const __grid_constant__ CUtensorMap tmap_x) {
  using L = SmemLayout<WFMT, BN, NP_, NA, NB>;
  constexpr int NP = NP_ > 0 ? NP_ : 1;   // ring size used in index math (no pack ring for f16 weights)
  constexpr int PACK = PackBytes<WFMT>::v;
  constexpr uint32_t NCOLS = BN < 32 ? 32 : BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem + L::a_off;
  uint8_t* sB = smem + L::b_off;
  uint8_t* sP = smem + L::p_off;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::bar_off);
  uint64_t* pack_full = bars;
  uint64_t* pack_empty = pack_full + NP_;
  uint64_t* a_full = pack_empty + NP_;
  uint64_t* a_empty = a_full + NA;
  uint64_t* b_full = a_empty + NA;
  uint64_t* b_empty = b_full + NB;
  uint64_t* acc_full = b_empty + NB;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mt = blockIdx.x, nt = blockIdx.y;
  const int S = gridDim.z, z = blockIdx.z;
  const int ks0 = (int)(((long long)z * p.ks_total) / S);
  const int ks1 = (int)(((long long)(z + 1) * p.ks_total) / S);
  const int nks = ks1 - ks0;

  if (threadIdx.x == 0) {
    for (int i = 0; i < NP_; ++i) { mbar_init(&pack_full[i], 1); mbar_init(&pack_empty[i], 8); }
    for (int i = 0; i < NA; ++i) { mbar_init(&a_full[i], WFMT == VG_WF_F16 ? 1 : 8); mbar_init(&a_empty[i], 1); }
    for (int i = 0; i < NB; ++i) { mbar_init(&b_full[i], 1); mbar_init(&b_empty[i], 1); }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, NCOLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int i = 0; i < nks && !*abort_flag; ++i) {
        const int ks = ks0 + i;
        if (WFMT != VG_WF_F16) {
          const int s = i % NP;
          if (!mbar_wait(&pack_empty[s], ((i / NP) & 1) ^ 1)) { report(p.err, VG_ERR_EMPTY_WAIT, abort_flag); break; }
          mbar_arrive_expect_tx(&pack_full[s], PACK);
          tma_bulk_g2s(sP + (size_t)s * PACK, p.wt + ((size_t)mt * p.ks_total + ks) * PACK, PACK, &pack_full[s]);
        } else {
          const int a = i % NA;
          if (!mbar_wait(&a_empty[a], ((i / NA) & 1) ^ 1)) { report(p.err, VG_ERR_EMPTY_WAIT, abort_flag); break; }
          mbar_arrive_expect_tx(&a_full[a], A_BYTES);
          tma_bulk_g2s(sA + (size_t)a * A_BYTES, p.wt + ((size_t)mt * p.ks_total + ks) * A_BYTES, A_BYTES, &a_full[a]);
        }
        const int b = i % NB;
        if (!mbar_wait(&b_empty[b], ((i / NB) & 1) ^ 1)) { report(p.err, VG_ERR_EMPTY_WAIT, abort_flag); break; }
        mbar_arrive_expect_tx(&b_full[b], L::b_bytes);
        uint8_t* bdst = sB + (size_t)b * L::b_bytes;
        tma_tensor2d_g2s(bdst, &tmap_x, ks * BK, nt * BN, &b_full[b]);
        tma_tensor2d_g2s(bdst + BN * 128, &tmap_x, ks * BK + 64, nt * BN, &b_full[b]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_f16(BM, BN, 0, 0);
      bool ok = true;
      for (int i = 0; i < nks && !*abort_flag; ++i) {
        const int a = i % NA, b = i % NB;
        if (!mbar_wait(&a_full[a], (i / NA) & 1)) { report(p.err, VG_ERR_DEQ_WAIT, abort_flag); ok = false; break; }
        if (!mbar_wait(&b_full[b], (i / NB) & 1)) { report(p.err, VG_ERR_TMA_WAIT, abort_flag); ok = false; break; }
        tc_fence_after();
        const uint32_t a_addr = smem_u32(sA + (size_t)a * A_BYTES);
        const uint32_t b_addr = smem_u32(sB + (size_t)b * L::b_bytes);
#pragma unroll
        for (int sub = 0; sub < 2; ++sub) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint64_t ad = umma_desc_sw128(a_addr + sub * SUB_BYTES + kk * 32);
            const uint64_t bd = umma_desc_sw128(b_addr + sub * (BN * 128) + kk * 32);
            umma_f16(tmem_base, ad, bd, idesc, (i | sub | kk) != 0 ? 1u : 0u);
          }
        }
        umma_commit(&a_empty[a]);
        umma_commit(&b_empty[b]);
      }
      if (ok) umma_commit(acc_full);
    }
  } else {
    // ------------------------------------------------ dequantizers
    if (WFMT != VG_WF_F16) {
      const int dt = threadIdx.x - 64;
      const int dw = dt >> 5;
      const int r = dw * 16 + (lane & 7) + ((lane >> 4) << 3);
      const int half = (lane >> 3) & 1;
      const int rs = r & 7;
      for (int i = 0; i < nks && !*abort_flag; ++i) {
        const int s = i % NP, a = i % NA;
        if (!mbar_wait(&pack_full[s], (i / NP) & 1)) { report(p.err, VG_ERR_TMA_WAIT, abort_flag); break; }
        if (!mbar_wait(&a_empty[a], ((i / NA) & 1) ^ 1)) { report(p.err, VG_ERR_EMPTY_WAIT, abort_flag); break; }
        const uint8_t* pk = sP + (size_t)s * PACK;
        uint8_t* arow = sA + (size_t)a * A_BYTES + half * SUB_BYTES + r * 128;
        if (WFMT == VG_WF_NVFP4) {
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
          *reinterpret_cast<uint4*>(arow + ((0 ^ rs) << 4)) = dequant8_fp4(p0.x, sc0);
          *reinterpret_cast<uint4*>(arow + ((1 ^ rs) << 4)) = dequant8_fp4(p0.y, sc0);
          *reinterpret_cast<uint4*>(arow + ((2 ^ rs) << 4)) = dequant8_fp4(p0.z, sc1);
          *reinterpret_cast<uint4*>(arow + ((3 ^ rs) << 4)) = dequant8_fp4(p0.w, sc1);
          *reinterpret_cast<uint4*>(arow + ((4 ^ rs) << 4)) = dequant8_fp4(p1.x, sc2);
          *reinterpret_cast<uint4*>(arow + ((5 ^ rs) << 4)) = dequant8_fp4(p1.y, sc2);
          *reinterpret_cast<uint4*>(arow + ((6 ^ rs) << 4)) = dequant8_fp4(p1.z, sc3);
          *reinterpret_cast<uint4*>(arow + ((7 ^ rs) << 4)) = dequant8_fp4(p1.w, sc3);
        } else {
          // FP8: row r holds 128 code bytes in eight 16-byte chunks stored at chunk ^ (r & 7).
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int j = half * 4 + c;     // source chunk: k = j*16 .. j*16+15
            const uint4 q = *reinterpret_cast<const uint4*>(pk + r * 128 + ((j ^ rs) << 4));
            uint4 lo, hi;
            lo.x = cvt_e4m3x2_f16x2((uint16_t)(q.x & 0xffff)); lo.y = cvt_e4m3x2_f16x2((uint16_t)(q.x >> 16));
            lo.z = cvt_e4m3x2_f16x2((uint16_t)(q.y & 0xffff)); lo.w = cvt_e4m3x2_f16x2((uint16_t)(q.y >> 16));
            hi.x = cvt_e4m3x2_f16x2((uint16_t)(q.z & 0xffff)); hi.y = cvt_e4m3x2_f16x2((uint16_t)(q.z >> 16));
            hi.z = cvt_e4m3x2_f16x2((uint16_t)(q.w & 0xffff)); hi.w = cvt_e4m3x2_f16x2((uint16_t)(q.w >> 16));
            *reinterpret_cast<uint4*>(arow + (((2 * c) ^ rs) << 4)) = lo;
            *reinterpret_cast<uint4*>(arow + (((2 * c + 1) ^ rs) << 4)) = hi;
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&a_full[a]);
          mbar_arrive(&pack_empty[s]);
        }
      }
    }
  }

  // ---------------------------------------------------- epilogue (warps 2..9)
  constexpr int CPW = BN / 2;            // accumulator columns handled by one warp
  float acc[CPW];
  bool have_acc = false;
  const int q = warp & 3;                // TMEM lane quarter this warp may read
  const int grp = warp >= 6 ? 1 : 0;     // which half of the columns
  const int m_local = q * 32 + lane;
  if (warp >= 2) {
    if (mbar_wait(acc_full, 0)) {
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < CPW; c += 8) {
        uint32_t v[8];
        tmem_ld8(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(grp * CPW + c), v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[c + j] = __uint_as_float(v[j]);
      }
      have_acc = true;
    } else {
      report(p.err, VG_ERR_MMA_WAIT, abort_flag);
    }
  }
  if (S > 1) {
    // Partial tiles go through distributed shared memory; cluster rank 0 sums them in rank order.
    float* red = reinterpret_cast<float*>(sA);
    if (warp >= 2 && have_acc) {
#pragma unroll
      for (int c = 0; c < CPW; ++c) red[(grp * CPW + c) * BM + m_local] = acc[c];
    }
    cluster_sync_all();
    if (z == 0 && warp >= 2 && have_acc) {
      const uint32_t red_addr = smem_u32(red);
      for (int s = 1; s < S; ++s) {
        const uint32_t remote = dsmem_map(red_addr, (uint32_t)s);
#pragma unroll
        for (int c = 0; c < CPW; ++c) acc[c] += dsmem_ld_f32(remote + (uint32_t)(((grp * CPW + c) * BM + m_local) * 4));
      }
    }
    cluster_sync_all();
  }
  if (warp >= 2 && have_acc && z == 0) {
    const int m = mt * BM + m_local;
    if (m < p.M) {
      const float rsc = p.row_scale ? p.row_scale[m] : 1.0f;
#pragma unroll
      for (int c = 0; c < CPW; ++c) {
        const int n = nt * BN + grp * CPW + c;
        if (n < p.N) {
          const float v = acc[c] * rsc;
          if (p.out_f32) reinterpret_cast<float*>(p.out)[(size_t)n * p.ldo + m] = v;
          else reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)n * p.ldo + m] = __float2bfloat16_rn(v);
        }
      }
    }
  }
  if (*abort_flag && threadIdx.x == 0) {
    // Give bulk copies that may still be in flight time to land before shared memory is released.
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, NCOLS);
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
std::map<TmapKey, CUtensorMap> g_tmaps;
std::mutex g_tmap_mu;

// Tensor map over X [rows, K] f16, row stride ldx elements; box = 64 k-elements x BN rows, 128-byte swizzle.
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

template <int WFMT, int BN, int NP, int NA, int NB>
int launch(const GemmParams& p, const CUtensorMap& tm, int splitk, cudaStream_t st) {
  using L = SmemLayout<WFMT, BN, NP, NA, NB>;
  auto kern = gemm_tc_kernel<WFMT, BN, NP, NA, NB>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::total);
    if (e != cudaSuccess) return (int)e;
    cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((p.M + BM - 1) / BM, (p.N + BN - 1) / BN, splitk);
  cfg.blockDim = dim3(320);
  cfg.dynamicSmemBytes = L::total;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = splitk;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, kern, p, tm);
}

template <int WFMT>
int dispatch_bn(const GemmParams& p, const void* x, int x_rows, int ldx, int splitk, cudaStream_t st) {
  CUtensorMap tm;
  int bn = p.N <= 16 ? 16 : (p.N <= 32 ? 32 : (p.N <= 64 ? 64 : 128));
  int rc = get_tmap_x(x, x_rows, p.K, bn, ldx, &tm);
  if (rc) return rc;
  constexpr bool F16 = WFMT == VG_WF_F16;
  switch (bn) {
    case 16: return launch<WFMT, 16, F16 ? 0 : 3, F16 ? 3 : 2, 3>(p, tm, splitk, st);
    case 32: return launch<WFMT, 32, F16 ? 0 : 3, F16 ? 3 : 2, 3>(p, tm, splitk, st);
    case 64: return launch<WFMT, 64, F16 ? 0 : 3, F16 ? 3 : 2, 3>(p, tm, splitk, st);
    default: return launch<WFMT, 128, F16 ? 0 : 3, F16 ? 3 : 2, 3>(p, tm, splitk, st);
  }
}

}  // namespace

extern "C" int vg_gemm_tc(const void* wt, const float* row_scale, const void* x_f16, int x_rows, int ldx, void* out,
                          int out_f32, int M, int K, int N, int ldo, int wfmt, int splitk, int* err,
                          cudaStream_t stream) {
  if (M <= 0 || K <= 0 || N <= 0 || (K % 16) != 0 || splitk < 1 || splitk > 8) return -2;
  if (ldx < K || (ldx % 8) != 0 || (reinterpret_cast<uintptr_t>(x_f16) & 15) != 0) return -4;
  GemmParams p;
  p.wt = static_cast<const uint8_t*>(wt);
  p.row_scale = row_scale;
  p.out = out;
  p.M = M; p.K = K; p.N = N; p.ldo = ldo;
  p.ks_total = (K + BK - 1) / BK;
  p.out_f32 = out_f32;
  p.err = err;
  if (splitk > p.ks_total) splitk = p.ks_total;
  if (N > 64) splitk = 1;
  switch (wfmt) {
    case VG_WF_NVFP4: return dispatch_bn<VG_WF_NVFP4>(p, x_f16, x_rows, ldx, splitk, stream);
    case VG_WF_FP8: return dispatch_bn<VG_WF_FP8>(p, x_f16, x_rows, ldx, splitk, stream);
    case VG_WF_F16: return dispatch_bn<VG_WF_F16>(p, x_f16, x_rows, ldx, splitk, stream);
  }
  return -3;
}

// Occupancy-derived number of CTAs of the decode configuration that can be resident at once (used by
// the host heuristic that picks the split-K factor).
extern "C" int vg_gemm_tc_resident_ctas(int wfmt) {
  int dev = 0, sms = 0, per_sm = 1;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (wfmt == VG_WF_NVFP4) {
    using L = SmemLayout<VG_WF_NVFP4, 16, 3, 2, 3>;
    auto kern = gemm_tc_kernel<VG_WF_NVFP4, 16, 3, 2, 3>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::total);
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, 320, L::total);
  }
  return sms * (per_sm > 0 ? per_sm : 1);
}

// GQA decode / verify attention on the 5th-generation tensor cores (head_dim 256, bf16 cache), split-K over keys.
//
// One CTA serves (column, KV head, split) for the WHOLE query group of the KV head, so each cache row is fetched
// once (the CUDA-core kernel in attention.cu launches one CTA per group of <= 4 query heads and refetches the rows
// for every group). Per 128-key tile:
//   S^T = K Q^T     tcgen05.mma kind::f16: A = the K tile as it lies in the cache ([key][dim], K-major, TMA with the
//                   128-byte swizzle), B = the group's query rows padded to 16; 128 x 16 fp32 accumulator in TMEM
//   softmax         four warps, thread = key: scale, mask, running maximum per head (warp shuffles + one exchange
//                   through shared memory), P written to shared memory as the bf16 B operand [head][key]
//   O^T += V^T P^T  A = the V tile used MN-major (dim is the M index, keys the contraction index: the cache layout
//                   [key][dim] is exactly that, so no transposed copy is needed), two M = 128 halves of the 256 dims
// K tiles travel through a two-slot ring and V tiles through one slot (64 KB each), filled by TMA from their own
// producer warps; S and P are double-buffered, and the issuer puts S(t+1) = K(t+1) Q^T ahead of O += V(t)^T P(t)^T, so
// the softmax of the next tile runs while the tensor core finishes the current one and the loads stay ahead of both. The split rule (a pure function of the column's own length), the partial-buffer format
// (max, sum, unnormalised accumulator per head and split) and the merge kernel are those of attention.cu, so a
// column's result does not depend on what else is in the batch (reference: kernels/gpu_batch.cu:1968-1975, :2132
// gqa_attn_splitk_gq reads each KV tile once per query group; this is the tensor-core form of that idea).
//
// Tiles are aligned to 128 keys and addressed through an optional block table (128-key pages): entry p of a
// column's table is the page holding its keys [128 p, 128 p + 128). Without a table the cache is the slotted layout
// [slot][kv head][max_seq][dim] and page p of a column is simply rows 128 p.. of its slot.
// All waits are bounded; a failed wait sets the error word and the CTA unwinds through the TMEM free.
#include <cuda.h>
#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"
#include "api.h"

namespace {
using namespace vg;

constexpr int HD = 256;
constexpr int BK = 128;                       // keys per tile
constexpr int SUB = 128 * 128;                // [128 rows x 64 bf16] swizzled sub-tile
constexpr int TILE = 4 * SUB;                 // 64 KB: one K or V tile
constexpr int NSLOT = 3;
constexpr int Q_BYTES = 4 * 2048;             // [16 heads][256 dims]: four [16 rows x 128 B] panels
constexpr int P_BYTES = 2 * 2048;             // [16 heads][128 keys]: two panels (two such buffers)
constexpr int SMEM_BYTES = NSLOT * TILE + Q_BYTES + 2 * P_BYTES + 1024 + 256 + 1024;
constexpr int THREADS = 224;                  // warp 0 K copies, warp 1 MMA issue, warps 2..5 softmax / epilogue, warp 6 V copies
constexpr uint32_t TM_S = 0, TM_O = 32, TM_COLS = 64;     // S: two 16-column buffers; O^T: two 16-column halves

VG_DEVINL void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
VG_DEVINL void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
VG_DEVINL void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// Shared-memory descriptor of an MN-major operand with the 128-byte swizzle: 64 consecutive M (or N) elements are one
// 128-byte row, eight rows (eight consecutive k) form a 1024-byte group (stride byte offset), the next 64 M elements
// start `lbo` bytes further (leading byte offset).
VG_DEVINL uint64_t umma_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)(lbo >> 4) << 16;
  d |= (uint64_t)(sbo >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

struct DecParams {
  const __nv_bfloat16* q;        // [N][nh][HD]
  const int* lens;
  const int* slots;
  const int* block_table;        // [N][bt_ld] page ids, or null (slotted cache)
  int bt_ld;
  float* part;                   // [N][nh][ns_grid][HD + 2]
  int nh, nkv, max_seq, ns_grid;
  float scale;
  int* err;
};

__device__ __forceinline__ int splits_for(int len, int ns_grid) {
  int ns = len / 64;
  ns = ns < 1 ? 1 : (ns > 32 ? 32 : ns);
  return ns > ns_grid ? ns_grid : ns;
}

__global__ void __launch_bounds__(THREADS, 1)
attn_decode_tc_kernel(const DecParams p, const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ring = smem;
  uint8_t* sQ = ring + NSLOT * TILE;
  uint8_t* sP = sQ + Q_BYTES;                                       // two P buffers
  float* xch = reinterpret_cast<float*>(sP + 2 * P_BYTES);         // [4 warps][16 heads] tile maxima, then sums
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * P_BYTES + 1024);
  uint64_t* k_full = bars;                // [2]
  uint64_t* k_empty = bars + 2;           // [2]
  uint64_t* v_full = bars + 4;
  uint64_t* v_empty = bars + 5;
  uint64_t* s_full = bars + 6;            // [2]
  uint64_t* p_ready = bars + 8;           // [2]
  uint64_t* pv_done = bars + 10;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  pdl_trigger();
  pdl_wait();
  const int len = p.lens[col];
  const int ns = splits_for(len, p.ns_grid);
  if (split >= ns) return;                                       // uniform for the CTA
  const int chunk = (len + ns - 1) / ns;
  const int k0 = split * chunk, k1 = min(len, k0 + chunk);
  const int page0 = k0 / BK;
  const int ntiles = k1 > k0 ? (k1 - 1) / BK - page0 + 1 : 0;
  const int G = p.nh / p.nkv, h0 = kvh * G;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); mbar_init(&s_full[i], 1); mbar_init(&p_ready[i], 128); }
    mbar_init(v_full, 1); mbar_init(v_empty, 1); mbar_init(pv_done, 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TM_COLS);
    tmem_relinquish();
  }
  // query rows of the group as the B operand [16][256] (rows >= G zero), and a zeroed P operand
  for (int c = threadIdx.x; c < 512; c += THREADS) {
    const int row = c >> 5, c16 = c & 31;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < G) v = *reinterpret_cast<const uint4*>(p.q + ((size_t)col * p.nh + h0 + row) * HD + c16 * 8);
    *reinterpret_cast<uint4*>(sQ + (c16 >> 3) * 2048 + row * 128 + (((c16 & 7) ^ (row & 7)) << 4)) = v;
  }
  for (int c = threadIdx.x; c < 2 * P_BYTES / 16; c += THREADS) reinterpret_cast<uint4*>(sP)[c] = make_uint4(0, 0, 0, 0);
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  auto fail = [&](int code) { if (p.err) atomicCAS(p.err, 0, code); *abort_flag = 1; };

  auto tile_row = [&](int t) -> int {
    const int page = page0 + t;
    if (p.block_table) return (int)(((long long)p.block_table[(size_t)col * p.bt_ld + page] * p.nkv + kvh) * BK);
    return (int)(((long long)p.slots[col] * p.nkv + kvh) * p.max_seq + (long long)page * BK);
  };
  if (warp == 0) {
    if (lane == 0) {                                         // K tiles: slots 0, 1 of the ring
      for (int t = 0; t < ntiles && !*abort_flag; ++t) {
        const int s = t & 1;
        if (!mbar_wait(&k_empty[s], ((t >> 1) & 1) ^ 1)) { fail(VG_ERR_EMPTY_WAIT); break; }
        uint8_t* dst = ring + (size_t)s * TILE;
        const int row0 = tile_row(t);
        mbar_arrive_expect_tx(&k_full[s], TILE);
#pragma unroll
        for (int j = 0; j < 4; ++j) tma_tensor2d_g2s(dst + j * SUB, &tm_k, 64 * j, row0, &k_full[s]);
      }
    }
  } else if (warp == 6) {
    if (lane == 0) {                                         // V tiles: slot 2
      for (int t = 0; t < ntiles && !*abort_flag; ++t) {
        if (!mbar_wait(v_empty, (t & 1) ^ 1)) { fail(VG_ERR_EMPTY_WAIT); break; }
        uint8_t* dst = ring + (size_t)2 * TILE;
        const int row0 = tile_row(t);
        mbar_arrive_expect_tx(v_full, TILE);
#pragma unroll
        for (int j = 0; j < 4; ++j) tma_tensor2d_g2s(dst + j * SUB, &tm_v, 64 * j, row0, v_full);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_f16(128, 16, 1, 1);                  // bf16 x bf16 -> fp32, K-major both
      constexpr uint32_t idesc_o = umma_idesc_f16(128, 16, 1, 1) | (1u << 15);     // A (the V tile) MN-major
      const uint64_t q_desc = umma_desc_sw128(smem_u32(sQ));
      const uint64_t v_desc = umma_desc_mn_sw128(smem_u32(ring + (size_t)2 * TILE), SUB, 1024);
      bool ok = true;
      auto issue_qk = [&](int t) -> bool {
        const int s = t & 1;
        if (!mbar_wait(&k_full[s], (t >> 1) & 1)) { fail(VG_ERR_TMA_WAIT); return false; }
        tc_fence_after();
        const uint64_t k_desc = umma_desc_sw128(smem_u32(ring + (size_t)s * TILE));
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk)
          umma_f16(tmem_base + TM_S + s * 16, k_desc + (uint64_t)(((kk >> 2) * SUB + (kk & 3) * 32) >> 4),
                   q_desc + (uint64_t)(((kk >> 2) * 2048 + (kk & 3) * 32) >> 4), idesc_s, kk ? 1u : 0u);
        umma_commit(&k_empty[s]);
        umma_commit(&s_full[s]);
        return true;
      };
      if (ntiles > 0) ok = issue_qk(0);
      for (int t = 0; t < ntiles && ok && !*abort_flag; ++t) {
        if (t + 1 < ntiles && !issue_qk(t + 1)) { ok = false; break; }            // S(t+1) ahead of O += V(t)^T P(t)^T
        if (!mbar_wait(&p_ready[t & 1], (t >> 1) & 1)) { fail(VG_ERR_MMA_WAIT); ok = false; break; }
        if (!mbar_wait(v_full, t & 1)) { fail(VG_ERR_TMA_WAIT); ok = false; break; }
        tc_fence_after();
        const uint64_t p_desc = umma_desc_sw128(smem_u32(sP + (t & 1) * P_BYTES));
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
          for (int ks = 0; ks < BK / 16; ++ks)
            umma_f16(tmem_base + TM_O + mt * 16, v_desc + (uint64_t)((mt * 2 * SUB + ks * 2048) >> 4),
                     p_desc + (uint64_t)(((ks >> 2) * 2048 + (ks & 3) * 32) >> 4), idesc_o, (t || ks) ? 1u : 0u);
        umma_commit(v_empty);
        umma_commit(pv_done);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax / epilogue: thread = key of the tile
    const int qd = warp & 3;                                 // TMEM lane quarter this warp may touch
    const int r = qd * 32 + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(qd * 32) << 16);
    float m_run[16], l_run[16];
#pragma unroll
    for (int h = 0; h < 16; ++h) { m_run[h] = -INFINITY; l_run[h] = 0.f; }
    bool ok = true;
    for (int t = 0; t < ntiles && ok && !*abort_flag; ++t) {
      if (!mbar_wait(&s_full[t & 1], (t >> 1) & 1)) { fail(VG_ERR_MMA_WAIT); ok = false; break; }
      tc_fence_after();
      const int key = (page0 + t) * BK + r;
      const bool valid = key >= k0 && key < k1;
      uint8_t* sPt = sP + (t & 1) * P_BYTES;
      uint32_t sv[16];
      tmem_ld16(lane_base + TM_S + (t & 1) * 16, sv);
      tmem_ld_wait();
      float s[16];
#pragma unroll
      for (int h = 0; h < 16; ++h) {
        if (h < G) {                                           // uniform: G is the same for every thread
          s[h] = valid ? __uint_as_float(sv[h]) * p.scale : -INFINITY;
          const float wm = warp_max(s[h]);
          if (lane == 0) xch[qd * 16 + h] = wm;
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      float corr[16];
      bool moved = false;
#pragma unroll
      for (int h = 0; h < 16; ++h) {
        corr[h] = 1.0f;
        if (h >= G) continue;
        const float mt_ = fmaxf(fmaxf(xch[h], xch[16 + h]), fmaxf(xch[32 + h], xch[48 + h]));
        const float m_new = fmaxf(m_run[h], mt_);
        corr[h] = m_new == -INFINITY ? 1.0f : __expf(m_run[h] - m_new);
        moved = moved || corr[h] != 1.0f;
        float pv = (valid && m_new != -INFINITY) ? __expf(s[h] - m_new) : 0.f;
        const __nv_bfloat16 pb = __float2bfloat16_rn(pv);
        // the sum runs over the rounded values the tensor core will multiply with
        l_run[h] = l_run[h] * corr[h] + __bfloat162float(pb);
        m_run[h] = m_new;
        *reinterpret_cast<__nv_bfloat16*>(sPt + (r >> 6) * 2048 + h * 128 + ((((r & 63) >> 3) ^ (h & 7)) << 4) + (r & 7) * 2) = pb;
      }
      // The previous tile's P V must have completed before O^T is rescaled (and it implies the one before, whose P
      // buffer this tile has just rewritten, completed too: that was awaited one tile ago).
      if (t > 0) {
        if (!mbar_wait(pv_done, (t - 1) & 1)) { fail(VG_ERR_MMA_WAIT); ok = false; break; }
        tc_fence_after();
      }
      // rescale O^T when some head's maximum moved (uniform: every thread sees the same maxima)
      if (t > 0 && moved) {
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
          uint32_t v[16];
          tmem_ld16(lane_base + TM_O + mt * 16, v);
          tmem_ld_wait();
#pragma unroll
          for (int h = 0; h < 16; ++h) v[h] = __float_as_uint(__uint_as_float(v[h]) * corr[h]);
          tmem_st16(lane_base + TM_O + mt * 16, v);
        }
        tmem_st_wait();
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&p_ready[t & 1]);
      asm volatile("bar.sync 1, 128;" ::: "memory");          // xch is rewritten by the next tile
    }
    if (ok && !*abort_flag && ntiles > 0) {
      if (!mbar_wait(pv_done, (ntiles - 1) & 1)) { fail(VG_ERR_MMA_WAIT); ok = false; }
    }
    if (ok && !*abort_flag) {
      tc_fence_after();
      // per-head sums over the 128 key threads
#pragma unroll
      for (int h = 0; h < 16; ++h) {
        if (h < G) {
          const float ws = warp_sum(l_run[h]);
          if (lane == 0) xch[qd * 16 + h] = ws;
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        uint32_t v[16];
        if (ntiles > 0) { tmem_ld16(lane_base + TM_O + mt * 16, v); tmem_ld_wait(); }
        const int d = mt * 128 + r;
        for (int h = 0; h < G; ++h) {
          float* pp = p.part + (((size_t)col * p.nh + h0 + h) * p.ns_grid + split) * (HD + 2);
          pp[2 + d] = ntiles > 0 ? __uint_as_float(v[h]) : 0.f;
          if (d == 0) {
            pp[0] = m_run[h];
            pp[1] = (xch[h] + xch[16 + h]) + (xch[32 + h] + xch[48 + h]);
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
  if (warp == 1) tmem_dealloc(tmem_base, TM_COLS);
}

// ------------------------------------------------------------------ host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_dec() {
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
std::map<std::tuple<const void*, long long>, CUtensorMap> g_dec_maps;
std::mutex g_dec_mu;

// [rows][256] bf16 row-major, boxes of 64 dims x 128 rows, 128-byte swizzle
int rows_map(const void* base, long long rows, CUtensorMap* out) {
  std::lock_guard<std::mutex> lk(g_dec_mu);
  auto key = std::make_tuple(base, rows);
  auto it = g_dec_maps.find(key);
  if (it != g_dec_maps.end()) { *out = it->second; return 0; }
  EncodeTiledFn enc = get_encode_dec();
  if (!enc) return -1;
  cuuint64_t dims[2] = {HD, (cuuint64_t)rows};
  cuuint64_t str[1] = {(cuuint64_t)HD * 2};
  cuuint32_t box[2] = {64, BK};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap tm;
  CUresult r = enc(&tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, str, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -(int)r - 100;
  if (g_dec_maps.size() > 1024) g_dec_maps.clear();
  g_dec_maps[key] = tm;
  *out = tm;
  return 0;
}
}  // namespace

int vg_attn_merge_launch(const float* part, const int* lens, int N, int nh, int hd, int ns_grid, const void* gate, int ld_gate,
                         void* out, cudaStream_t st);

// Tensor-core split-K decode attention + merge. kc / vc: bf16 cache of `cache_rows` rows of 256 values: the slotted
// layout [slots][nkv][max_seq][256] (block_table null), or a page pool [pages][nkv][128][256] addressed through
// block_table [N][bt_ld] (entry p = page of the column's keys [128 p, 128 p + 128)). Other arguments as vg_attn_decode.
// The query group nh / nkv must be <= 16.
extern "C" int vg_attn_decode_tc(const void* q, const void* kc, const void* vc, long long cache_rows, const int* lens,
                                 const int* slots, const int* block_table, int bt_ld, float* part, int N, int nh, int nkv, int hd,
                                 int max_seq, int ns_grid, const void* gate, int ld_gate, void* out, int* err, cudaStream_t st) {
  if (N <= 0) return 0;
  if (hd != HD || nh % nkv != 0 || nh / nkv > 16 || ns_grid < 1 || ns_grid > 32 || (!block_table && !slots)) return -2;
  CUtensorMap tk, tv;
  int rc = rows_map(kc, cache_rows, &tk);
  if (rc) return rc;
  rc = rows_map(vc, cache_rows, &tv);
  if (rc) return rc;
  DecParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.lens = lens; p.slots = slots; p.block_table = block_table; p.bt_ld = bt_ld;
  p.part = part;
  p.nh = nh; p.nkv = nkv; p.max_seq = max_seq; p.ns_grid = ns_grid;
  p.scale = rsqrtf((float)HD);
  p.err = err;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  cudaError_t e = launch_pdl(attn_decode_tc_kernel, dim3(N, nkv, ns_grid), dim3(THREADS), SMEM_BYTES, st, p, tk, tv);
  if (e != cudaSuccess) return (int)e;
  // (A merge by the last-arriving split inside this launch was measured and rejected: one CTA pulling a KV head's
  // 6 x 32 partial rows through L2 takes longer (+37 us) than the separate, fully parallel merge launch costs.)
  return vg_attn_merge_launch(part, lens, N, nh, hd, ns_grid, gate, ld_gate, out, st);
}

// Causal GQA attention for prefill on the 5th-generation tensor cores (head_dim 256, bf16).
//
// One CTA per (128-query tile, query head). Per 128-key tile:
//   S = Q K^T      tcgen05.mma kind::f16 (bf16 operands from shared memory, 128 x 128 fp32 accumulator in TMEM)
//   softmax        four warps, thread = query row: online max / sum in fp32 read from TMEM with tcgen05.ld,
//                  causal mask on the diagonal tile, O rescaled in TMEM only when a row maximum moved
//   O += P V       P is written back to TMEM as bf16 (tcgen05.st) and used as the A operand (TS form), V comes
//                  from a transposed copy of the lane's values ([kv head][dim][key], K-major for the B operand)
// Q / K / V^T tiles arrive by tiled TMA copies with the 128-byte swizzle (3-D maps over the slotted cache, no
// multicast); K and V have their own full / empty barriers so the next K loads under the softmax and the next
// V under the next S. The epilogue normalises, applies the sigmoid output gate and writes the f16 input of
// o_proj. Keys are the lane's cache rows [0, pos0 + n): earlier prefill chunks are attended through the cache.
// (reference: kernels/gpu_batch.cu:1078-1083, :1238-1324 do this phase with scalar / warp-MMA kernels.)
//
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
constexpr int BQ = 128;                      // queries per CTA
constexpr int BKV = 128;                     // keys per tile
constexpr int SUB = 128 * 128;               // bytes of one [128 rows x 64 bf16] swizzled sub-tile
constexpr int Q_BYTES = BQ * HD * 2;         // 65536: 4 sub-tiles along the head dim
constexpr int K_BYTES = BKV * HD * 2;        // 65536
constexpr int V_BYTES = HD * BKV * 2;        // 65536: 2 sub-tiles of [256 dims x 64 keys]
constexpr int VSUB = HD * 128;               // bytes of one [256 rows x 64 bf16] sub-tile
constexpr int SMEM_BYTES = Q_BYTES + K_BYTES + V_BYTES + 16 * 8 + 16 + 1024;
constexpr int THREADS = 192;                 // warp 0 copies, warp 1 issues MMAs, warps 2..5 softmax / epilogue
constexpr uint32_t TM_S = 0, TM_O = 128, TM_P = 384, TM_COLS = 512;

VG_DEVINL void tma_tensor3d_g2s(void* smem_dst, const void* tmap, int c0, int c1, int c2, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
          smem_u32(smem_dst)),
      "l"(tmap), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar))
      : "memory");
}
VG_DEVINL void tmem_ld32(uint32_t taddr, uint32_t* r) {
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
VG_DEVINL void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
VG_DEVINL void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
VG_DEVINL void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

struct PfParams {
  const __nv_bfloat16* gate;     // fused qkv rows (gate of head h at h*2*HD + HD), or null
  int ld_gate;
  __half* out;                   // [n][nh*HD]
  int nh, nkv, pos0, n;
  float scale_log2;              // softmax scale * log2(e)
  int* err;
};

__global__ void __launch_bounds__(THREADS, 1)
attn_prefill_kernel(const PfParams p, const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + Q_BYTES;
  uint8_t* sV = sK + K_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + V_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = bars + 2;
  uint64_t* v_full = bars + 3;
  uint64_t* v_empty = bars + 4;
  uint64_t* s_full = bars + 5;
  uint64_t* p_ready = bars + 6;
  uint64_t* o_done = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * BQ;
  const int head = blockIdx.y;
  const int kvh = head / (p.nh / p.nkv);
  const int q_last = min(q0 + BQ, p.n) - 1;                 // last valid query row of this tile
  const int nkt = (p.pos0 + q_last) / BKV + 1;              // key tiles that hold a visible key
  pdl_trigger();

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1); mbar_init(k_full, 1); mbar_init(k_empty, 1); mbar_init(v_full, 1); mbar_init(v_empty, 1);
    mbar_init(s_full, 1); mbar_init(p_ready, 128); mbar_init(o_done, 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  auto fail = [&](int code) { if (p.err) atomicCAS(p.err, 0, code); *abort_flag = 1; };

  if (warp == 0) {
    if (lane == 0) {
      pdl_wait();
      mbar_arrive_expect_tx(q_full, Q_BYTES);
#pragma unroll
      for (int j = 0; j < 4; ++j) tma_tensor2d_g2s(sQ + j * SUB, &tm_q, head * HD + 64 * j, q0, q_full);
      for (int t = 0; t < nkt && !*abort_flag; ++t) {
        if (!mbar_wait(k_empty, (t & 1) ^ 1)) { fail(VG_ERR_EMPTY_WAIT); break; }
        mbar_arrive_expect_tx(k_full, K_BYTES);
#pragma unroll
        for (int j = 0; j < 4; ++j) tma_tensor3d_g2s(sK + j * SUB, &tm_k, 64 * j, t * BKV, kvh, k_full);
        if (!mbar_wait(v_empty, (t & 1) ^ 1)) { fail(VG_ERR_EMPTY_WAIT); break; }
        mbar_arrive_expect_tx(v_full, V_BYTES);
#pragma unroll
        for (int j = 0; j < 2; ++j) tma_tensor3d_g2s(sV + j * VSUB, &tm_v, t * BKV + 64 * j, 0, kvh, v_full);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_f16(BQ, BKV, 1, 1);       // bf16 x bf16 -> fp32, N = 128
      constexpr uint32_t idesc_o = umma_idesc_f16(BQ, HD, 1, 1);        // N = 256
      const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK), v_addr = smem_u32(sV);
      bool ok = mbar_wait(q_full, 0);
      if (!ok) fail(VG_ERR_TMA_WAIT);
      for (int t = 0; t < nkt && ok && !*abort_flag; ++t) {
        if (!mbar_wait(k_full, t & 1)) { fail(VG_ERR_TMA_WAIT); ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk)
          umma_f16(tmem_base + TM_S, umma_desc_sw128(q_addr + (kk >> 2) * SUB + (kk & 3) * 32),
                   umma_desc_sw128(k_addr + (kk >> 2) * SUB + (kk & 3) * 32), idesc_s, kk ? 1u : 0u);
        umma_commit(k_empty);
        umma_commit(s_full);
        if (!mbar_wait(p_ready, t & 1)) { fail(VG_ERR_MMA_WAIT); ok = false; break; }
        if (!mbar_wait(v_full, t & 1)) { fail(VG_ERR_TMA_WAIT); ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk)
          umma_bf16_ts(tmem_base + TM_O, tmem_base + TM_P + (uint32_t)kk * 8,
                       umma_desc_sw128(v_addr + (kk >> 2) * VSUB + (kk & 3) * 32), idesc_o, (t || kk) ? 1u : 0u);
        umma_commit(v_empty);
        if (t == nkt - 1) umma_commit(o_done);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax / epilogue: thread = query row
    const int qd = warp & 3;                               // TMEM lane quarter this warp may touch
    const int r = qd * 32 + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(qd * 32) << 16);
    const int qpos = p.pos0 + q0 + r;                      // absolute position of this row's query
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int t = 0; t < nkt && ok && !*abort_flag; ++t) {
      if (!mbar_wait(s_full, t & 1)) { fail(VG_ERR_MMA_WAIT); ok = false; break; }
      tc_fence_after();
      const bool diag = (t + 1) * BKV - 1 > p.pos0 + q0;    // some key of the tile may lie beyond some query
      // pass 1: row maximum of the tile
      float mx = -INFINITY;
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) {
        uint32_t v[32];
        tmem_ld32(lane_base + TM_S + c4 * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int key = t * BKV + c4 * 32 + i;
          const float s = __uint_as_float(v[i]) * p.scale_log2;
          mx = fmaxf(mx, (diag && key > qpos) ? -INFINITY : s);
        }
      }
      const float m_new = fmaxf(m_run, mx);
      const float corr = m_new == -INFINITY ? 1.0f : exp2f(m_run - m_new);
      // pass 2: probabilities -> bf16 A operand in TMEM
      float lsum = 0.f;
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        uint32_t pk[32];
#pragma unroll
        for (int c2 = 0; c2 < 2; ++c2) {
          uint32_t v[32];
          tmem_ld32(lane_base + TM_S + (h2 * 2 + c2) * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const int key = t * BKV + (h2 * 2 + c2) * 32 + i;
            float p0 = exp2f(__uint_as_float(v[i]) * p.scale_log2 - m_new);
            float p1 = exp2f(__uint_as_float(v[i + 1]) * p.scale_log2 - m_new);
            if (m_new == -INFINITY || (diag && key > qpos)) p0 = 0.f;
            if (m_new == -INFINITY || (diag && key + 1 > qpos)) p1 = 0.f;
            const __nv_bfloat162 b2 = __floats2bfloat162_rn(p0, p1);
            // the sum runs over the rounded values the tensor core will multiply with
            lsum += __bfloat162float(b2.x) + __bfloat162float(b2.y);
            pk[c2 * 16 + (i >> 1)] = *reinterpret_cast<const uint32_t*>(&b2);
          }
        }
        tmem_st32(lane_base + TM_P + h2 * 32, pk);
      }
      // rescale O only when some row of this warp moved its maximum (the previous P V has completed: MMAs
      // retire in order and this tile's S came after it)
      if (t > 0 && __any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t v[32];
          tmem_ld32(lane_base + TM_O + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * corr);
          tmem_st32(lane_base + TM_O + c * 32, v);
        }
      }
      tmem_st_wait();
      l_run = l_run * corr + lsum;
      m_run = m_new;
      tc_fence_before();
      mbar_arrive(p_ready);
    }
    // ---------------------------------------------------------------- epilogue
    if (ok && !*abort_flag) {
      if (!mbar_wait(o_done, 0)) { fail(VG_ERR_MMA_WAIT); ok = false; }
    }
    if (ok && !*abort_flag) {
      tc_fence_after();
      pdl_wait();
      const int row = q0 + r;
      const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(lane_base + TM_O + c * 32, v);
        tmem_ld_wait();
        if (row < p.n) {
          __half* dst = p.out + ((size_t)row * p.nh + head) * HD + c * 32;
          const __nv_bfloat16* gp = p.gate ? p.gate + (size_t)row * p.ld_gate + (size_t)head * 2 * HD + HD + c * 32 : nullptr;
#pragma unroll
          for (int i8 = 0; i8 < 4; ++i8) {
            uint4 o4;
            __half* h = reinterpret_cast<__half*>(&o4);
            uint4 g4 = make_uint4(0, 0, 0, 0);
            if (gp) g4 = *reinterpret_cast<const uint4*>(gp + i8 * 8);
            const __nv_bfloat16* gb = reinterpret_cast<const __nv_bfloat16*>(&g4);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              float o = __uint_as_float(v[i8 * 8 + i]) * inv;
              if (gp) o *= sigmoidf(__bfloat162float(gb[i]));
              h[i] = f32_to_f16_sat(o);
            }
            *reinterpret_cast<uint4*>(dst + i8 * 8) = o4;
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

// vT[kvh][d][t] = vc[slot][kvh][t][d] for t < len (32 x 32 tiles through shared memory).
__global__ void transpose_v_kernel(const __nv_bfloat16* __restrict__ v, __nv_bfloat16* __restrict__ vT, int max_seq, int len,
                                   int vt_cap) {
  __shared__ __nv_bfloat16 tile[32][33];
  pdl_trigger();
  pdl_wait();
  const int kvh = blockIdx.z, t0 = blockIdx.x * 32, d0 = blockIdx.y * 32;
  const __nv_bfloat16* src = v + (size_t)kvh * max_seq * HD;
  __nv_bfloat16* dst = vT + (size_t)kvh * HD * vt_cap;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int t = t0 + i;
    tile[i][threadIdx.x] = t < len ? src[(size_t)t * HD + d0 + threadIdx.x] : __float2bfloat16(0.f);
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int t = t0 + threadIdx.x;
    if (t < vt_cap) dst[(size_t)(d0 + i) * vt_cap + t] = tile[threadIdx.x][i];
  }
}

// 4-bit cache -> bf16 staging for the tensor-core kernel: rows[kvh][t][d] and / or transposed[kvh][d][t], t < len
// (zeros up to the end of the last 128-key tile in the transposed copy).
__global__ void kv_q4_dequant_kernel(const uint8_t* __restrict__ codes, const __half* __restrict__ scales,
                                     __nv_bfloat16* __restrict__ rows, __nv_bfloat16* __restrict__ tr, int hd, int max_seq,
                                     int len, int t_cap) {
  __shared__ __nv_bfloat16 tile[32][33];
  pdl_trigger();
  pdl_wait();
  const int kvh = blockIdx.z, t0 = blockIdx.x * 32, d0 = blockIdx.y * 32;
  const uint8_t* cs = codes + (size_t)kvh * max_seq * (hd / 2);
  const __half* ss = scales + (size_t)kvh * max_seq * (hd / 16);
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int t = t0 + i, d = d0 + threadIdx.x;
    float v = 0.f;
    if (t < len) {
      const uint8_t b = cs[(size_t)t * (hd / 2) + (d >> 1)];
      const int code = (d & 1) ? (b >> 4) : (b & 15);
      v = (float)(code - 8) * __half2float(ss[(size_t)t * (hd / 16) + (d >> 4)]);
    }
    const __nv_bfloat16 o = __float2bfloat16_rn(v);
    tile[i][threadIdx.x] = o;
    if (rows && t < len) rows[((size_t)kvh * max_seq + t) * hd + d] = o;
  }
  if (!tr) return;
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int t = t0 + threadIdx.x;
    if (t < t_cap) tr[((size_t)kvh * hd + d0 + i) * t_cap + t] = tile[threadIdx.x][i];
  }
}

// ------------------------------------------------------------------ host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_pf() {
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
using MapKey = std::tuple<const void*, long long, long long, long long, int>;
std::map<MapKey, CUtensorMap> g_maps;
std::mutex g_mu;

// rank-2 or rank-3 bf16 map with the 128-byte swizzle; dims / strides innermost first (strides in bytes, rank-1 of them)
int make_map(const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides, const cuuint32_t* box, CUtensorMap* out) {
  std::lock_guard<std::mutex> lk(g_mu);
  MapKey key{base, (long long)dims[0], (long long)dims[1], rank == 3 ? (long long)dims[2] : 0, (int)box[1] * 4 + rank};
  auto it = g_maps.find(key);
  if (it != g_maps.end()) { *out = it->second; return 0; }
  EncodeTiledFn enc = get_encode_pf();
  if (!enc) return -1;
  cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMap tm;
  CUresult r = enc(&tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -(int)r - 100;
  if (g_maps.size() > 1024) g_maps.clear();
  g_maps[key] = tm;
  *out = tm;
  return 0;
}
}  // namespace

// Transposed copy of one lane's cached values: vT [nkv][256][vt_cap] <- vc [slot][nkv][max_seq][256], rows < len.
extern "C" int vg_attn_transpose_v(const void* vc, void* vT, int slot, int nkv, int hd, int max_seq, int len, int vt_cap,
                                   cudaStream_t st) {
  if (hd != HD || len > vt_cap || (vt_cap % 64) != 0) return -2;
  if (len <= 0) return 0;
  const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(vc) + (size_t)slot * nkv * max_seq * HD;
  const int tcols = (((len + 127) / 128) * 128 + 31) / 32;        // whole key tiles are written (zeros beyond len)
  launch_pdl(transpose_v_kernel, dim3(tcols, HD / 32, nkv), dim3(32, 8), 0, st, src, static_cast<__nv_bfloat16*>(vT), max_seq, len,
             vt_cap);
  return (int)cudaGetLastError();
}

// One lane's 4-bit cache rows [0, len) -> bf16: `out_rows` [nkv][max_seq][hd] (same row pitch as the cache, so it
// can stand in for a one-slot bf16 cache) and / or `out_transposed` [nkv][hd][t_cap]; either may be null.
extern "C" int vg_kv_q4_dequant(const void* codes, const void* scales, int slot, int nkv, int hd, int max_seq, int len,
                                void* out_rows, void* out_transposed, int t_cap, cudaStream_t st) {
  if ((hd % 32) != 0 || len > max_seq || (out_transposed && len > t_cap)) return -2;
  if (len <= 0) return 0;
  const uint8_t* c = static_cast<const uint8_t*>(codes) + (size_t)slot * nkv * max_seq * (hd / 2);
  const __half* sc = static_cast<const __half*>(scales) + (size_t)slot * nkv * max_seq * (hd / 16);
  const int tcols = (((len + 127) / 128) * 128 + 31) / 32;
  launch_pdl(kv_q4_dequant_kernel, dim3(tcols, hd / 32, nkv), dim3(32, 8), 0, st, c, sc, static_cast<__nv_bfloat16*>(out_rows),
             static_cast<__nv_bfloat16*>(out_transposed), hd, max_seq, len, t_cap);
  return (int)cudaGetLastError();
}

// q [q_cap][nh*256] bf16 (rows < n valid), keys / values = cache rows [0, pos0 + n) of `slot`; vT from
// vg_attn_transpose_v. Writes out [n][nh*256] f16 (gated when `gate` is given, as the decode merge kernel does).
extern "C" int vg_attn_prefill_tc(const void* q, int q_cap, const void* kc, const void* vT, int vt_cap, int slot, int nkv,
                                  int nh, int hd, int max_seq, int pos0, int n, float scale, const void* gate, int ld_gate,
                                  void* out_f16, int* err, cudaStream_t st) {
  if (hd != HD || n <= 0 || nh % nkv != 0 || pos0 + n > max_seq || ((pos0 + n + 127) / 128) * 128 > vt_cap || (ld_gate % 8) != 0)
    return -2;
  CUtensorMap tq, tk, tv;
  {
    cuuint64_t dims[2] = {(cuuint64_t)nh * HD, (cuuint64_t)q_cap};
    cuuint64_t str[1] = {(cuuint64_t)nh * HD * 2};
    cuuint32_t box[2] = {64, BQ};
    int rc = make_map(q, 2, dims, str, box, &tq);
    if (rc) return rc;
  }
  {
    const __nv_bfloat16* kb = static_cast<const __nv_bfloat16*>(kc) + (size_t)slot * nkv * max_seq * HD;
    cuuint64_t dims[3] = {HD, (cuuint64_t)max_seq, (cuuint64_t)nkv};
    cuuint64_t str[2] = {(cuuint64_t)HD * 2, (cuuint64_t)max_seq * HD * 2};
    cuuint32_t box[3] = {64, BKV, 1};
    int rc = make_map(kb, 3, dims, str, box, &tk);
    if (rc) return rc;
  }
  {
    cuuint64_t dims[3] = {(cuuint64_t)vt_cap, HD, (cuuint64_t)nkv};
    cuuint64_t str[2] = {(cuuint64_t)vt_cap * 2, (cuuint64_t)HD * vt_cap * 2};
    cuuint32_t box[3] = {64, HD, 1};
    int rc = make_map(vT, 3, dims, str, box, &tv);
    if (rc) return rc;
  }
  PfParams p;
  p.gate = static_cast<const __nv_bfloat16*>(gate);
  p.ld_gate = ld_gate;
  p.out = static_cast<__half*>(out_f16);
  p.nh = nh; p.nkv = nkv; p.pos0 = pos0; p.n = n;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.err = err;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return (int)launch_pdl(attn_prefill_kernel, dim3((n + BQ - 1) / BQ, nh), dim3(THREADS), SMEM_BYTES, st, p, tq, tk, tv);
}

// GatedDeltaNet kernels: depthwise causal conv (k <= 8) + SiLU, and the gated delta-rule recurrence
// with the gated RMSNorm fused in. Decode, width-N verify (chain, tree, multi-lane forest) and prefill
// all run the SAME per-token arithmetic in the SAME order, so verify(N) is bit-identical to N decodes
// (reference: kernels/gpu_batch.cu:405-418, :439-660, :1326-1440 get this the same way, with separate
// decode and prefill kernels that share the scalar recurrence).
//
// Column bookkeeping (device int arrays, one entry per token column):
//   in_slot[t]   state slot holding the lane's state before its first column
//   parent[t]    column whose output state this column continues from, or -1 (start from in_slot[t])
//   out_slot[t]  state slot that receives the state after this column, or -1
// Decode: parent = -1, out_slot = in_slot. Chain verify: parent = t-1, out_slot = checkpoint slots.
// Prefill: parent = t-1, out_slot = -1 except the last column.
//
// Recurrence kernel: one CTA per (value head, chain); thread j owns column j of the head's state
// S[kd, vd] in registers, so the three kd-long dot products are thread-local sequential sums and need
// no cross-thread reduction. State layout [slot][nv][kd][vd] fp32; conv state [slot][conv_dim][ck] fp32
// with the newest sample last.
#include "common.cuh"
#include "act_quant.cuh"
#include "api.h"

namespace {
using namespace vg;

constexpr int MAX_CK = 8;

__global__ void gdn_conv_kernel(const __nv_bfloat16* __restrict__ x, int ldx, float* __restrict__ state,
                                const float* __restrict__ w, const int* __restrict__ in_slot,
                                const int* __restrict__ parent, const int* __restrict__ out_slot,
                                float* __restrict__ out, int N, int conv_dim, int ck, int phase, int t_first) {
  if (threadIdx.x == 0) trace(80);
  pdl_trigger();
  pdl_wait();
  if (threadIdx.x == 0) trace(81);
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)(N - t_first) * conv_dim) return;
  const int t = t_first + (int)(idx / conv_dim), c = (int)(idx % conv_dim);
  const int os = out_slot[t];
  if (!(phase & 1) && os < 0) return;
  float win[MAX_CK];
  int cur = t, j = ck - 1;
  for (; j >= 0 && cur >= 0; --j) {
    win[j] = __bfloat162float(x[(size_t)cur * ldx + c]);
    cur = parent[cur];
  }
  const int d = ck - 1 - j;                 // samples taken from the columns
  const float* st = state + ((size_t)in_slot[t] * conv_dim + c) * ck;
  for (int jj = j; jj >= 0; --jj) win[jj] = st[jj + d];
  if (phase & 1) {
    float acc = 0.f;
    for (int i = 0; i < ck; ++i) acc = fmaf(w[(size_t)c * ck + i], win[i], acc);
    out[(size_t)t * conv_dim + c] = silu(acc);
  }
  if ((phase & 2) && os >= 0) {
    float* dst = state + ((size_t)os * conv_dim + c) * ck;
    for (int i = 0; i < ck; ++i) dst[i] = win[i];
  }
}

// Prefill form of the conv for one linear chain (parent[t] = t - 1, token 0 continues the state of in_slot[0]):
// a thread owns eight adjacent channels and walks TS consecutive tokens with the window in registers, so every
// input row is read once with 16-byte loads instead of ck times with 2-byte loads. Same taps in the same
// ascending FMA order as gdn_conv_kernel. Conv + SiLU only: the state update of the chain's last token runs
// afterwards as gdn_conv_kernel phase 2 over that token (it must not overlap the reads of the old state here).
template <int CK, int TS>
__global__ void __launch_bounds__(128) gdn_conv_chain_kernel(const __nv_bfloat16* __restrict__ x, int ldx,
                                                             const float* __restrict__ state, const float* __restrict__ w,
                                                             const int* __restrict__ in_slot, float* __restrict__ out, int N,
                                                             int conv_dim) {
  pdl_trigger();
  // the taps do not depend on the preceding kernel
  const int c = ((int)blockIdx.x * 128 + (int)threadIdx.x) * 8;
  const bool live = c < conv_dim;
  float wt[8][CK];
  if (live) {
#pragma unroll
    for (int k = 0; k < 8; ++k)
#pragma unroll
      for (int i = 0; i < CK; ++i) wt[k][i] = w[(size_t)(c + k) * CK + i];
  }
  pdl_wait();
  if (!live) return;
  const int t_begin = (int)blockIdx.y * TS, t_end = min(t_begin + TS, N);
  float win[8][CK];       // win[k][CK - 1] is the current token's sample
  // history before t_begin: from the rows of earlier tokens, or from the carried state before token 0
#pragma unroll
  for (int i = 0; i < CK - 1; ++i) {
    const int t = t_begin - (CK - 1) + i;
    if (t >= 0) {
      const uint4 v = *reinterpret_cast<const uint4*>(x + (size_t)t * ldx + c);
      const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
      for (int k = 0; k < 8; ++k) win[k][i + 1] = __bfloat162float(b[k]);
    } else {
      // the state holds the last CK samples; sample of (virtual) token t is its entry CK + t
      const float* st = state + ((size_t)in_slot[0] * conv_dim + c) * CK;
#pragma unroll
      for (int k = 0; k < 8; ++k) win[k][i + 1] = st[(size_t)k * CK + (CK + t)];
    }
  }
#pragma unroll 4
  for (int t = t_begin; t < t_end; ++t) {
    const uint4 v = *reinterpret_cast<const uint4*>(x + (size_t)t * ldx + c);
    const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(&v);
    float o[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
#pragma unroll
      for (int i = 0; i < CK - 1; ++i) win[k][i] = win[k][i + 1];
      win[k][CK - 1] = __bfloat162float(b[k]);
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < CK; ++i) acc = fmaf(wt[k][i], win[k][i], acc);
      o[k] = silu(acc);
    }
    float4* dst = reinterpret_cast<float4*>(out + (size_t)t * conv_dim + c);
    dst[0] = make_float4(o[0], o[1], o[2], o[3]);
    dst[1] = make_float4(o[4], o[5], o[6], o[7]);
  }
}

// col_ctr[t]: heads of column t counted in; [COL_AMAX + t]: running maximum of its outputs; [COL_DONE + t]: heads that
// have finished their share of the row (all-resident form)
constexpr int COL_AMAX = 16, COL_DONE = 32;

template <int KD, int VD>
__global__ void __launch_bounds__(VD) gdn_step_kernel(
    const float* __restrict__ qkv, const __nv_bfloat16* __restrict__ proj, int ldp, int off_z, int off_b, int off_a,
    float* __restrict__ S, const float* __restrict__ A_log, const float* __restrict__ dt_bias,
    const float* __restrict__ norm_w, const int* __restrict__ chain_start, const int* __restrict__ chain_len,
    const int* __restrict__ in_slot, const int* __restrict__ parent, const int* __restrict__ out_slot,
    __half* __restrict__ out, int nk, int nv, float eps, uint8_t* __restrict__ bq, int ldb, uint8_t* __restrict__ sfb,
    float* __restrict__ g0, unsigned int* __restrict__ col_ctr, int all_resident, int* __restrict__ err) {
  if (threadIdx.x == 0) trace(96);
  pdl_trigger();
  __shared__ float red[32];
  __shared__ float hs[VD];                // this head's outputs of the current column (all-resident row quantisation)
  __shared__ __align__(16) float ks[KD];
  __shared__ __align__(16) float qs[KD];
  __shared__ int is_last;
  const int vh = blockIdx.x, chain = blockIdx.y, j = threadIdx.x;
  const int kh = vh * nk / nv;
  const int key_dim = nk * KD, conv_dim = 2 * key_dim + nv * VD;
  // Per-head constants, the column bookkeeping (uploaded at the start of the step) and the lane's input state
  // (last written by the previous step) do not depend on the preceding kernel: fetch them before waiting for it.
  const int t0 = chain_start[chain], tn = chain_len[chain];
  const float a_coef = -__expf(A_log[vh]);
  const float dtb = dt_bias[vh];
  const float nw = norm_w[j];
  float s[KD];
  int loaded_from = -2;      // column whose output state is in registers (-2: nothing)
  const bool preloaded = tn > 0 && parent[t0] < 0;
  if (preloaded) {
    const float* sp = S + (((size_t)in_slot[t0] * nv + vh) * KD) * VD + j;
#pragma unroll
    for (int a = 0; a < KD; ++a) s[a] = sp[(size_t)a * VD];
  }
  pdl_wait();
  if (threadIdx.x == 0) trace(97);
  for (int t = t0; t < t0 + tn; ++t) {
    const int par = parent[t];
    if (t == t0 ? !preloaded : par != loaded_from) {
      const int src = par < 0 ? in_slot[t] : out_slot[par];
      const float* sp = S + (((size_t)src * nv + vh) * KD) * VD + j;
#pragma unroll
      for (int a = 0; a < KD; ++a) s[a] = sp[(size_t)a * VD];
    }
    // q, k of the key head: l2-normalise (eps 1e-6), q also scaled by 1/sqrt(kd)
    const float* row = qkv + (size_t)t * conv_dim;
    float qv = 0.f, kv = 0.f;
    // every global read of the column is issued here, ahead of the first barrier, so their latencies overlap
    const float v = row[2 * key_dim + vh * VD + j];
    const float bb = __bfloat162float(proj[(size_t)t * ldp + off_b + vh]);
    const float aa = __bfloat162float(proj[(size_t)t * ldp + off_a + vh]) + dtb;
    const float z = __bfloat162float(proj[(size_t)t * ldp + off_z + vh * VD + j]);
    for (int i = j; i < KD; i += VD) {
      qs[i] = row[kh * KD + i];
      ks[i] = row[key_dim + kh * KD + i];
    }
    __syncthreads();
    for (int i = j; i < KD; i += VD) { qv += qs[i] * qs[i]; kv += ks[i] * ks[i]; }
    const float qn = block_sum(qv, red);
    const float kn = block_sum(kv, red);
    const float qsc = rsqrtf(qn + 1e-6f) * rsqrtf((float)KD);
    const float ksc = rsqrtf(kn + 1e-6f);
    const float beta = sigmoidf(bb);
    const float sp_ = aa > 20.f ? aa : log1pf(__expf(aa));
    const float g = __expf(a_coef * sp_);
    // decay + kv_mem. Canonical summation order (shared with the prefill kernel, where four threads split a
    // column): each quarter of the key range keeps four interleaved partial sums; the quarters are added
    // pairwise, (q0 + q1) + (q2 + q3).
    constexpr int HK = KD / 4;
    float hsum[4];
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      float m0 = 0.f, m1 = 0.f, m2 = 0.f, m3 = 0.f;
#pragma unroll
      for (int a = h * HK; a < (h + 1) * HK; a += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(&ks[a]);
        s[a] *= g; s[a + 1] *= g; s[a + 2] *= g; s[a + 3] *= g;
        m0 = fmaf(s[a], k4.x, m0); m1 = fmaf(s[a + 1], k4.y, m1);
        m2 = fmaf(s[a + 2], k4.z, m2); m3 = fmaf(s[a + 3], k4.w, m3);
      }
      hsum[h] = (m0 + m1) + (m2 + m3);
    }
    const float kv_mem = ((hsum[0] + hsum[1]) + (hsum[2] + hsum[3])) * ksc;
    const float delta = (v - kv_mem) * beta;
    const float dk = delta * ksc;
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
      for (int a = h * HK; a < (h + 1) * HK; a += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(&ks[a]);
        const float4 q4 = *reinterpret_cast<const float4*>(&qs[a]);
        s[a] = fmaf(k4.x, dk, s[a]); s[a + 1] = fmaf(k4.y, dk, s[a + 1]);
        s[a + 2] = fmaf(k4.z, dk, s[a + 2]); s[a + 3] = fmaf(k4.w, dk, s[a + 3]);
        o0 = fmaf(s[a], q4.x, o0); o1 = fmaf(s[a + 1], q4.y, o1);
        o2 = fmaf(s[a + 2], q4.z, o2); o3 = fmaf(s[a + 3], q4.w, o3);
      }
      hsum[h] = (o0 + o1) + (o2 + o3);
    }
    const float o = ((hsum[0] + hsum[1]) + (hsum[2] + hsum[3])) * qsc;
    const float ss = block_sum(o * o, red);
    const __half o16 = f32_to_f16_sat(o * rsqrtf(ss / (float)VD + eps) * nw * silu(z));
    out[((size_t)t * nv + vh) * VD + j] = o16;
    const int os = out_slot[t];
    if (os >= 0) {
      float* dp = S + (((size_t)os * nv + vh) * KD) * VD + j;
#pragma unroll
      for (int a = 0; a < KD; ++a) dp[(size_t)a * VD] = s[a];
    }
    loaded_from = t;
    if (threadIdx.x == 0) trace(6 * 16 + 3);
    bool tail = false;
    if (bq) {
      // The output projection reads this row as the FP4 series, which needs the row's maximum (over all heads)
      // before any block can be quantised. Every head folds the maximum of its own outputs into the column's running
      // maximum (non-negative floats order like their bit patterns) and then counts itself in.
      //  * all_resident (the grid fits on the GPU at once, so no CTA waits for one that cannot start): every head
      //    waits (bounded) until all heads of the column are counted, then quantises its own VD outputs, so the row
      //    is quantised by nv CTAs side by side; the last head to finish zeroes the column's words.
      //  * otherwise the head counted in last quantises the whole row, reading it back through L2.
      // Both forms run the same arithmetic on the same values: the bits do not depend on the form.
      const float hmax = aq::block_max(fabsf(__half2float(o16)), red);
      if (all_resident) hs[j] = __half2float(o16);
      __threadfence();
      __syncthreads();
      if (j == 0) {
        atomicMax(&col_ctr[COL_AMAX + t], __float_as_uint(hmax));
        __threadfence();
        is_last = atomicAdd(&col_ctr[t], 1u) == (unsigned)nv - 1u;
      }
      const int K = nv * VD, nblk = ldb >> 3;          // ldb bytes per row = Kpad / 2
      if (all_resident) {
        if (j == 0) {
          uint64_t t_start = 0;
          for (int tries = 0; ld_acquire_gpu(&col_ctr[t]) < (unsigned)nv; ++tries) {
            if (tries == 256) t_start = global_ns();
            if (tries > 256 && (tries & 63) == 0 && global_ns() - t_start > 100000000ull) {    // 100 ms: far beyond any skew between heads, short of a hang
              if (err) atomicCAS(err, 0, VG_ERR_GRID_WAIT);
              break;
            }
          }
        }
        __syncthreads();
        const float amax = __uint_as_float(__ldcg(&col_ctr[COL_AMAX + t]));
        const float gq = amax > 0.f ? amax / (6.0f * 448.0f) : 1.0f;
        if (vh == 0 && j == 0) g0[t] = gq;
        // this head's VD / 16 blocks; head 0 also writes the zero blocks that pad the row to the GEMM's K
        constexpr int HB = VD / 16;
        const int pad0 = K >> 4;
        int b = -1;
        if (j < HB) b = vh * HB + j;
        else if (vh == 0 && pad0 + (j - HB) < nblk) b = pad0 + (j - HB);
        if (b >= 0) {
          float r[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) r[i] = j < HB ? hs[j * 16 + i] : 0.f;
          aq::quant_block(r, gq, t, b, bq, ldb, sfb);
        }
        __syncthreads();
        if (j == 0 && atomicAdd(&col_ctr[COL_DONE + t], 1u) == (unsigned)nv - 1u) {
          col_ctr[t] = 0; col_ctr[COL_AMAX + t] = 0; col_ctr[COL_DONE + t] = 0;     // every head has read the maximum
        }
      } else {
      __syncthreads();
      tail = is_last != 0;
      if (tail) {
        if (threadIdx.x == 0) trace(6 * 16 + 4);
        __threadfence();
        const __half* row16 = out + (size_t)t * K;
        const float amax = __uint_as_float(__ldcg(&col_ctr[COL_AMAX + t]));
        const float gq = amax > 0.f ? amax / (6.0f * 448.0f) : 1.0f;
        if (j == 0) g0[t] = gq;
        constexpr int PF = 4;                            // blocks whose loads are in flight together
        for (int b0 = j; b0 < nblk; b0 += PF * VD) {
          uint4 u[PF][2];
#pragma unroll
          for (int q = 0; q < PF; ++q) {
            const int b = b0 + q * VD;
            if (b < nblk && b * 16 < K) {
              u[q][0] = __ldcg(reinterpret_cast<const uint4*>(row16 + b * 16));
              u[q][1] = __ldcg(reinterpret_cast<const uint4*>(row16 + b * 16) + 1);
            } else {
              u[q][0] = make_uint4(0, 0, 0, 0);
              u[q][1] = make_uint4(0, 0, 0, 0);
            }
          }
#pragma unroll
          for (int q = 0; q < PF; ++q) {
            const int b = b0 + q * VD;
            if (b >= nblk) break;
            float r[16];
            const __half2* h0 = reinterpret_cast<const __half2*>(&u[q][0]);
            const __half2* h1 = reinterpret_cast<const __half2*>(&u[q][1]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 a = __half22float2(h0[i]), c = __half22float2(h1[i]);
              r[2 * i] = a.x; r[2 * i + 1] = a.y; r[8 + 2 * i] = c.x; r[8 + 2 * i + 1] = c.y;
            }
            aq::quant_block(r, gq, t, b, bq, ldb, sfb);
          }
        }
      }
      }
    }
    __syncthreads();   // qs/ks are rewritten by the next column
    if (tail && j == 0) trace(6 * 16 + 5);
    if (tail && j == 0) { col_ctr[t] = 0; col_ctr[COL_AMAX + t] = 0; }   // every thread of the tail has read the maximum
  }
  if (threadIdx.x == 0) trace(6 * 16 + 2);
}

}  // namespace

extern "C" int vg_gdn_conv(const void* x, int ldx, float* state, const float* w, const int* in_slot, const int* parent,
                           const int* out_slot, float* out, int N, int conv_dim, int ck, int phase, cudaStream_t st) {
  if (N <= 0) return 0;
  if (ck > MAX_CK) return -2;
  const size_t total = (size_t)N * conv_dim;
  launch_pdl(gdn_conv_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, st, static_cast<const __nv_bfloat16*>(x), ldx, state, w,
                                                                   in_slot, parent, out_slot, out, N, conv_dim, ck, phase, 0);
  return (int)cudaGetLastError();
}

// Conv + SiLU + state update of one linear chain of N tokens (parent[t] = t - 1; only the last token has an
// output slot): the prefill form of vg_gdn_conv phases 1 + 2. Returns -2 for shapes it does not cover.
extern "C" int vg_gdn_conv_chain(const void* x, int ldx, float* state, const float* w, const int* in_slot, const int* parent,
                                 const int* out_slot, float* out, int N, int conv_dim, int ck, cudaStream_t st) {
  if (N <= 0) return 0;
  if (ck != 4 || (conv_dim % 8) != 0 || (ldx % 8) != 0 || ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) != 0)
    return -2;
  constexpr int TS = 16;
  launch_pdl(gdn_conv_chain_kernel<4, TS>, dim3((unsigned)((conv_dim / 8 + 127) / 128), (unsigned)((N + TS - 1) / TS)), dim3(128), 0, st,
             static_cast<const __nv_bfloat16*>(x), ldx, (const float*)state, w, in_slot, out, N, conv_dim);
  // state of the last token (the only one with an output slot)
  launch_pdl(gdn_conv_kernel, dim3((unsigned)((conv_dim + 255) / 256)), dim3(256), 0, st, static_cast<const __nv_bfloat16*>(x), ldx, state, w,
             in_slot, parent, out_slot, out, N, conv_dim, ck, 2, N - 1);
  return (int)cudaGetLastError();
}

namespace {
using namespace vg;

// ------------------------------------------------------------------ prefill: one long chain per CTA
// Same arithmetic, in the same order, as gdn_step_kernel applied token by token (so a prefilled state is
// bit-identical to stepping through the prompt), restructured so the per-token critical path is only the
// thread-local FMA chains: tokens arrive in batches of TB through a double-buffered cp.async ring, the three
// block-wide reductions of a token (|q|^2, |k|^2, |o|^2) are computed for a whole batch at once by the warps
// with the exact shuffle tree block_sum uses, and there is one barrier pair per batch instead of seven per
// token. Linear chains only (parent[t] = t - 1).
VG_DEVINL void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
VG_DEVINL void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
VG_DEVINL void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// block_sum(v) of a VD-thread block whose thread c holds x[c], reproduced by one warp (VD == 128).
template <int VD>
VG_DEVINL float block_sum_by_warp(const float* x, int lane) {
  float p[VD / 32];
#pragma unroll
  for (int w = 0; w < VD / 32; ++w) p[w] = warp_sum(x[32 * w + lane]);
  float r = 0.f;
#pragma unroll
  for (int w = 0; w < VD / 32; ++w) r = lane == w ? p[w] : r;
  return warp_sum(r);
}

// Packed pairs of fp32 (sm_100 f32x2 arithmetic): one instruction performs two IEEE fp32 operations, so the
// results are the bits of the scalar form while the recurrence issues half as many FMA-pipe instructions.
VG_DEVINL uint64_t pk2(float a, float b) { uint64_t r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b)); return r; }
VG_DEVINL void upk2(uint64_t v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
VG_DEVINL uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
VG_DEVINL uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

// CS CTAs share one value head, each owning VD / CS state columns (the kernel stalls on shared-memory latency
// with one CTA per head, and only nv SMs would be busy). With CS > 1 the gated output norm, the only step that
// couples a head's columns, moves to gdn_out_norm_kernel: this kernel then stores the raw outputs (fp32).
template <int KD, int VD, int TB, int CS, int TPC>
__global__ void __launch_bounds__(TPC * VD / CS) gdn_prefill_kernel(
    const float* __restrict__ qkv, const __nv_bfloat16* __restrict__ proj, int ldp, int off_z, int off_b, int off_a,
    float* __restrict__ S, const float* __restrict__ A_log, const float* __restrict__ dt_bias,
    const float* __restrict__ norm_w, int t0, int tn, const int* __restrict__ in_slot, const int* __restrict__ out_slot,
    __half* __restrict__ out, float* __restrict__ o_raw, int nk, int nv, float eps) {
  constexpr int VC = VD / CS;              // state columns of this CTA
  // TPC threads share a state column, each owning QPT of the four quarters of the key range (the quarters are
  // the unit of the canonical summation order). In shared memory every quarter of a q / k row is followed by a
  // 16-byte pad, so the TPC different 16-byte reads of a warp's load instruction fall into different banks.
  constexpr int QK = KD / 4, QPT = 4 / TPC;
  constexpr int KDP = KD + 16;             // padded q / k row
  constexpr int NT = TPC * VC, NWARP = NT / 32, HK = KD / TPC;
  static_assert(KD == VD && VD % 32 == 0 && VC % 32 == 0 && TB % NWARP == 0 && KD % 16 == 0, "layout");
  static_assert(TPC == 2 || TPC == 4, "threads per column");
  extern __shared__ __align__(16) float sm[];
  float* qb = sm;                          // [2][TB][KDP] raw q
  float* kb = qb + 2 * TB * KDP;           // [2][TB][KDP] raw k
  float* vb = kb + 2 * TB * KDP;           // [2][TB][VC]
  float* ob = vb + 2 * TB * VC;            // [TB][VC]    o before the output norm
  float* sq = ob + TB * VC;                // [TB][VC]    o^2 staging for the batched reductions
  float* sc = sq + TB * VC;                // [TB][4]     g, beta, ksc, qsc
  float* ssb = sc + TB * 4;                // [TB]        sum o^2
  float* bab = ssb + TB;                   // [TB][2]     b, a of the batch (as float)
  int* osl = reinterpret_cast<int*>(bab + TB * 2);                       // [TB] out_slot
  __nv_bfloat16* zb = reinterpret_cast<__nv_bfloat16*>(osl + TB);        // [2][TB][VC] gate z (CS == 1 only)
  pdl_trigger();
  pdl_wait();
  const int vh = blockIdx.x / CS, part = blockIdx.x % CS;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cl = tid / TPC, h = tid % TPC; // local column and which quarter of the key range
  const int c = part * VC + cl;            // column of the head's state
  const int kh = vh * nk / nv;
  const int key_dim = nk * KD, conv_dim = 2 * key_dim + nv * VD;
  const float a_coef = -__expf(A_log[vh]);
  const float dtb = dt_bias[vh];
  const float nw = norm_w[c];
  constexpr int TPW = TB / NWARP;          // tokens per warp in the batched phases

  uint64_t s2[HK / 2];                     // state elements (2i, 2i + 1) of this thread's key range
  {
    const float* sp = S + (((size_t)in_slot[t0] * nv + vh) * KD + h * HK) * VD + c;
#pragma unroll
    for (int a = 0; a < HK; a += 2) s2[a / 2] = pk2(sp[(size_t)a * VD], sp[(size_t)(a + 1) * VD]);
  }
  auto issue = [&](int b) {                // batch b -> buffer b & 1
    const int base = t0 + b * TB, cnt = min(TB, tn - b * TB);
    float* q_ = qb + (b & 1) * TB * KDP;
    float* k_ = kb + (b & 1) * TB * KDP;
    float* v_ = vb + (b & 1) * TB * VC;
    __nv_bfloat16* z_ = zb + (b & 1) * TB * VC;
    constexpr int CPT = KD / 4;            // 16-byte chunks per fp32 q / k row
    for (int i = tid; i < cnt * CPT; i += NT) {
      const int tt = i / CPT, o4 = (i % CPT) * 4;
      const float* row = qkv + (size_t)(base + tt) * conv_dim;
      const int po = o4 + (o4 / QK) * 4;   // padded offset
      cp_async16(q_ + tt * KDP + po, row + kh * KD + o4);
      cp_async16(k_ + tt * KDP + po, row + key_dim + kh * KD + o4);
    }
    constexpr int CPV = VC / 4;
    for (int i = tid; i < cnt * CPV; i += NT) {
      const int tt = i / CPV, o4 = (i % CPV) * 4;
      cp_async16(v_ + tt * VC + o4, qkv + (size_t)(base + tt) * conv_dim + 2 * key_dim + vh * VD + part * VC + o4);
    }
    if (CS == 1) {
      constexpr int CPZ = VC / 8;          // 16-byte chunks per bf16 z row
      for (int i = tid; i < cnt * CPZ; i += NT) {
        const int tt = i / CPZ, o8 = (i % CPZ) * 8;
        cp_async16(z_ + tt * VC + o8, proj + (size_t)(base + tt) * ldp + off_z + vh * VD + o8);
      }
    }
    cp_async_commit();
  };
  // b / a / out_slot of a batch: fetched one batch ahead into registers by the first TB threads
  float nb_b = 0.f, nb_a = 0.f;
  int nb_os = -1;
  auto fetch_scalars = [&](int b) {
    const int tt = tid;
    if (tt < TB && b * TB + tt < tn) {
      const int t = t0 + b * TB + tt;
      nb_b = __bfloat162float(proj[(size_t)t * ldp + off_b + vh]);
      nb_a = __bfloat162float(proj[(size_t)t * ldp + off_a + vh]);
      nb_os = out_slot[t];
    }
  };
  const int nb = (tn + TB - 1) / TB;
  if (nb > 0) { issue(0); fetch_scalars(0); }
  for (int b = 0; b < nb; ++b) {
    const int base = t0 + b * TB, cnt = min(TB, tn - b * TB);
    const float* q_ = qb + (b & 1) * TB * KDP;
    const float* k_ = kb + (b & 1) * TB * KDP;
    const float* v_ = vb + (b & 1) * TB * VC;
    const __nv_bfloat16* z_ = zb + (b & 1) * TB * VC;
    if (tid < TB) { bab[tid * 2] = nb_b; bab[tid * 2 + 1] = nb_a; osl[tid] = nb_os; }
    cp_async_wait_all();
    __syncthreads();                       // batch b landed; everyone is done with batch b - 1
    if (b + 1 < nb) { issue(b + 1); fetch_scalars(b + 1); }
    // ---- per-token scalars of the batch (warp w: tokens w*TPW ..), block_sum order reproduced per warp
    for (int u = 0; u < TPW; ++u) {
      const int tt = warp * TPW + u;
      if (tt >= cnt) break;
      float pq[VD / 32], pk[VD / 32];
#pragma unroll
      for (int w = 0; w < VD / 32; ++w) {
        const int pi = 32 * w + lane + ((32 * w + lane) / QK) * 4;
        const float x = q_[tt * KDP + pi], y = k_[tt * KDP + pi];
        pq[w] = warp_sum(x * x);
        pk[w] = warp_sum(y * y);
      }
      float rq = 0.f, rk = 0.f;
#pragma unroll
      for (int w = 0; w < VD / 32; ++w) { rq = lane == w ? pq[w] : rq; rk = lane == w ? pk[w] : rk; }
      const float qn = warp_sum(rq), kn = warp_sum(rk);
      if (lane == 0) {
        const float bb = bab[tt * 2];
        const float aa = bab[tt * 2 + 1] + dtb;
        const float sp_ = aa > 20.f ? aa : log1pf(__expf(aa));
        sc[tt * 4 + 0] = __expf(a_coef * sp_);
        sc[tt * 4 + 1] = sigmoidf(bb);
        sc[tt * 4 + 2] = rsqrtf(kn + 1e-6f);
        sc[tt * 4 + 3] = rsqrtf(qn + 1e-6f) * rsqrtf((float)KD);
      }
    }
    __syncthreads();
    // ---- the recurrence: thread-local FMA chains, one shuffle per dot product
    for (int tt = 0; tt < cnt; ++tt) {
      const float g = sc[tt * 4 + 0], beta = sc[tt * 4 + 1], ksc = sc[tt * 4 + 2], qsc = sc[tt * 4 + 3];
      const float* ks = k_ + tt * KDP + h * QPT * (QK + 4);
      const float* qs = q_ + tt * KDP + h * QPT * (QK + 4);
      const float v = v_[tt * VC + cl];
      // this thread's part of k stays in registers (as pairs) for both passes over the state
      uint64_t kr[HK / 2];
#pragma unroll
      for (int qq = 0; qq < QPT; ++qq)
#pragma unroll
        for (int a = 0; a < QK; a += 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(&ks[qq * (QK + 4) + a]);
          kr[(qq * QK + a) / 2] = pk2(k4.x, k4.y);
          kr[(qq * QK + a) / 2 + 1] = pk2(k4.z, k4.w);
        }
      const uint64_t g2 = pk2(g, g);
      float part[QPT];
#pragma unroll
      for (int qq = 0; qq < QPT; ++qq) {
        uint64_t m01 = pk2(0.f, 0.f), m23 = pk2(0.f, 0.f);     // the four interleaved partial sums, as two pairs
#pragma unroll
        for (int a = qq * QK; a < (qq + 1) * QK; a += 4) {
          s2[a / 2] = mul2(s2[a / 2], g2);
          s2[a / 2 + 1] = mul2(s2[a / 2 + 1], g2);
          m01 = fma2(s2[a / 2], kr[a / 2], m01);
          m23 = fma2(s2[a / 2 + 1], kr[a / 2 + 1], m23);
        }
        float m0, m1, m2, m3;
        upk2(m01, m0, m1);
        upk2(m23, m2, m3);
        part[qq] = (m0 + m1) + (m2 + m3);
      }
      // quarters (q0 + q1) + (q2 + q3): IEEE addition commutes, so every thread of the column gets the same bits
      float mine = QPT == 2 ? part[0] + part[QPT - 1] : part[0];
      mine += __shfl_xor_sync(0xffffffffu, mine, 1);
      if (TPC == 4) mine += __shfl_xor_sync(0xffffffffu, mine, 2);
      const float kv_mem = mine * ksc;
      const float delta = (v - kv_mem) * beta;
      const float dk = delta * ksc;
      const uint64_t dk2 = pk2(dk, dk);
#pragma unroll
      for (int qq = 0; qq < QPT; ++qq) {
        uint64_t o01 = pk2(0.f, 0.f), o23 = pk2(0.f, 0.f);
#pragma unroll
        for (int a = qq * QK; a < (qq + 1) * QK; a += 4) {
          const float4 q4 = *reinterpret_cast<const float4*>(&qs[qq * (QK + 4) + (a - qq * QK)]);
          s2[a / 2] = fma2(kr[a / 2], dk2, s2[a / 2]);
          s2[a / 2 + 1] = fma2(kr[a / 2 + 1], dk2, s2[a / 2 + 1]);
          o01 = fma2(s2[a / 2], pk2(q4.x, q4.y), o01);
          o23 = fma2(s2[a / 2 + 1], pk2(q4.z, q4.w), o23);
        }
        float o0, o1, o2, o3;
        upk2(o01, o0, o1);
        upk2(o23, o2, o3);
        part[qq] = (o0 + o1) + (o2 + o3);
      }
      mine = QPT == 2 ? part[0] + part[QPT - 1] : part[0];
      mine += __shfl_xor_sync(0xffffffffu, mine, 1);
      if (TPC == 4) mine += __shfl_xor_sync(0xffffffffu, mine, 2);
      const float o = mine * qsc;
      if (h == 0) {
        ob[tt * VC + cl] = o;
        if (CS == 1) sq[tt * VC + cl] = o * o;
      }
      const int os = osl[tt];
      if (os >= 0) {
        float* dp = S + (((size_t)os * nv + vh) * KD + h * HK) * VD + c;
#pragma unroll
        for (int a = 0; a < HK; a += 2) {
          float e0, e1;
          upk2(s2[a / 2], e0, e1);
          dp[(size_t)a * VD] = e0;
          dp[(size_t)(a + 1) * VD] = e1;
        }
      }
    }
    __syncthreads();
    if constexpr (CS > 1) {
      // raw outputs of the batch, coalesced; the norm over the whole head runs in gdn_out_norm_kernel
      for (int i = tid; i < cnt * VC; i += NT) {
        const int tt = i / VC, cc = i % VC;
        o_raw[((size_t)(base + tt) * nv + vh) * VD + part * VC + cc] = ob[tt * VC + cc];
      }
    } else {
      // ---- output norm of the batch
      for (int u = 0; u < TPW; ++u) {
        const int tt = warp * TPW + u;
        if (tt >= cnt) break;
        const float ss = block_sum_by_warp<VD>(sq + tt * VD, lane);
        if (lane == 0) ssb[tt] = ss;
      }
      __syncthreads();
      for (int tt = h; tt < cnt; tt += TPC) {
        const float z = __bfloat162float(z_[tt * VD + c]);
        out[((size_t)(base + tt) * nv + vh) * VD + c] =
            f32_to_f16_sat(ob[tt * VD + c] * rsqrtf(ssb[tt] / (float)VD + eps) * nw * silu(z));
      }
    }
  }
}

// Gated output norm of the column-split prefill: one warp per (token, head), eight per CTA. The sum of squares
// follows the step kernel's block_sum (per-warp butterflies over elements 32 w + lane, then a butterfly over the
// VD / 32 partials), so the results are the same bits.
template <int VD>
__global__ void __launch_bounds__(256) gdn_out_norm_kernel(const float* __restrict__ o_raw, const __nv_bfloat16* __restrict__ proj,
                                                           int ldp, int off_z, const float* __restrict__ norm_w, int t0, int tn,
                                                           __half* __restrict__ out, int nv, float eps) {
  constexpr int NW = VD / 32;
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const size_t item = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);      // (token, head) pair
  if (item >= (size_t)tn * nv) return;
  const int t = t0 + (int)(item / nv), vh = (int)(item % nv);
  const float* op = o_raw + ((size_t)t * nv + vh) * VD;
  const __nv_bfloat16* zp = proj + (size_t)t * ldp + off_z + vh * VD;
  float o[NW], z[NW], p[NW];
#pragma unroll
  for (int w = 0; w < NW; ++w) { o[w] = op[32 * w + lane]; z[w] = __bfloat162float(zp[32 * w + lane]); }
#pragma unroll
  for (int w = 0; w < NW; ++w) p[w] = warp_sum(o[w] * o[w]);
  float r = 0.f;
#pragma unroll
  for (int w = 0; w < NW; ++w) r = lane == w ? p[w] : r;
  const float ss = warp_sum(r);
  const float inv = rsqrtf(ss / (float)VD + eps);
  __half* dst = out + ((size_t)t * nv + vh) * VD;
#pragma unroll
  for (int w = 0; w < NW; ++w) dst[32 * w + lane] = f32_to_f16_sat(o[w] * inv * norm_w[32 * w + lane] * silu(z[w]));
}

}  // namespace

// bq / sfb / g0 / col_ctr (all or none): also emit each column's output row as the FP4 activation series for
// the output projection (at most 16 columns); col_ctr is 48 zero-initialised words (two counters and a running
// maximum per column) that the kernel leaves zeroed. `err` (may be null) receives VG_ERR_GRID_WAIT if the heads of a
// column waited too long for each other.
// Needs column index < 16, (nv * vd) % 16 == 0 and ldb * 2 >= nv * vd with ldb % 128 == 0.
extern "C" int vg_gdn_step(const float* qkv, const void* proj, int ldp, int off_z, int off_b, int off_a, float* S,
                           const float* A_log, const float* dt_bias, const float* norm_w, const int* chain_start,
                           const int* chain_len, int n_chains, const int* in_slot, const int* parent, const int* out_slot,
                           void* out_f16, int nk, int nv, int kd, int vd, float eps, void* bq, int ldb, void* sfb,
                           float* g0, unsigned int* col_ctr, int* err, cudaStream_t st) {
  if (n_chains <= 0) return 0;
  if (bq && (!sfb || !g0 || !col_ctr || (ldb % 128) != 0 || ldb * 2 < nv * vd || ((nv * vd) % 16) != 0)) return -2;
  dim3 grid(nv, n_chains);
  // Row quantisation by all heads side by side needs every CTA of the grid on the GPU at once (they wait for each
  // other): at most one CTA per SM is assumed, whatever else is resident. VELO_GDN_RESIDENT_QUANT=0 turns it off.
  static const bool resident_on = [] { const char* e = getenv("VELO_GDN_RESIDENT_QUANT"); return !(e && e[0] == '0'); }();
  static const int n_sm = [] {
    int dev = 0, n = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n;
  }();
  const int all_resident = (bq && resident_on && (long long)nv * n_chains <= n_sm) ? 1 : 0;
  const __nv_bfloat16* pj = static_cast<const __nv_bfloat16*>(proj);
  __half* o = static_cast<__half*>(out_f16);
  uint8_t* bqp = static_cast<uint8_t*>(bq);
  uint8_t* sfp = static_cast<uint8_t*>(sfb);
  if (kd == 128 && vd == 128)
    launch_pdl(gdn_step_kernel<128, 128>, dim3(grid), dim3(128), 0, st, qkv, pj, ldp, off_z, off_b, off_a, S, A_log, dt_bias, norm_w, chain_start, chain_len, in_slot, parent, out_slot, o, nk, nv, eps, bqp, ldb, sfp, g0, col_ctr, all_resident, err);
  else if (kd == 64 && vd == 64)
    launch_pdl(gdn_step_kernel<64, 64>, dim3(grid), dim3(64), 0, st, qkv, pj, ldp, off_z, off_b, off_a, S, A_log, dt_bias, norm_w, chain_start, chain_len, in_slot, parent, out_slot, o, nk, nv, eps, bqp, ldb, sfp, g0, col_ctr, all_resident, err);
  else
    return -3;
  return (int)cudaGetLastError();
}

// One linear chain of `tn` columns starting at column t0 (prefill): same results as vg_gdn_step on that chain.
// `o_scratch` (fp32, at least (t0 + tn) * nv * vd elements, or null) enables the column-split form: `split` CTAs
// per head (1, 2 or 4; 0 = pick so that the grid fills the SMs) plus a separate output-norm kernel.
extern "C" int vg_gdn_prefill(const float* qkv, const void* proj, int ldp, int off_z, int off_b, int off_a, float* S,
                              const float* A_log, const float* dt_bias, const float* norm_w, int t0, int tn,
                              const int* in_slot, const int* out_slot, void* out_f16, int nk, int nv, int kd, int vd,
                              float eps, float* o_scratch, int split, cudaStream_t st) {
  if (tn <= 0) return 0;
  if (kd != 128 || vd != 128) return -3;
  // 16-byte async copies: every staged row must start on a 16-byte boundary
  if ((ldp % 8) != 0 || (off_z % 8) != 0 || (reinterpret_cast<uintptr_t>(proj) & 15) || (reinterpret_cast<uintptr_t>(qkv) & 15))
    return -2;
  constexpr int TB = 16;
  if (split == 0) split = !o_scratch ? 1 : (nv * 4 <= 160 ? 4 : (nv * 2 <= 160 ? 2 : 1));
  if (split != 1 && (!o_scratch || (split != 2 && split != 4))) return -2;
  auto smem_for = [](int cs) {
    const int vc = 128 / cs;
    return (size_t)(2 * TB * (128 + 16) * 2 + 2 * TB * vc + 2 * TB * vc + TB * 4 + TB + TB * 2) * sizeof(float) + TB * sizeof(int) +
           (size_t)2 * TB * vc * sizeof(__nv_bfloat16);
  };
  const __nv_bfloat16* pj = static_cast<const __nv_bfloat16*>(proj);
  __half* o16 = static_cast<__half*>(out_f16);
#define VG_GDN_PF(CS, TPC)                                                                                                 \
  {                                                                                                                     \
    static bool configured = false;                                                                                     \
    if (!configured) {                                                                                                  \
      cudaError_t e = cudaFuncSetAttribute(gdn_prefill_kernel<128, 128, TB, CS, TPC>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           (int)smem_for(CS));                                                          \
      if (e != cudaSuccess) return (int)e;                                                                              \
      configured = true;                                                                                                \
    }                                                                                                                   \
    launch_pdl(gdn_prefill_kernel<128, 128, TB, CS, TPC>, dim3(nv * CS), dim3(TPC * 128 / CS), smem_for(CS), st, qkv, pj, ldp, off_z, off_b, \
               off_a, S, A_log, dt_bias, norm_w, t0, tn, in_slot, out_slot, o16, o_scratch, nk, nv, eps);                 \
  }
  // threads per state column: two keep a 64-column CTA at 128 threads; with a head split four ways (32-column
  // CTAs, the tensor-parallel case) four threads per column do the same (measured 1.26 -> 0.96 ms per layer)
  static const int tpc_env = [] { const char* e = getenv("VELO_GDN_PREFILL_TPC"); return e ? (e[0] == '4' ? 4 : 2) : 0; }();
  const int tpc = tpc_env ? tpc_env : (split == 4 ? 4 : 2);
  if (tpc == 4) {
    if (split == 4) VG_GDN_PF(4, 4)
    else if (split == 2) VG_GDN_PF(2, 4)
    else VG_GDN_PF(1, 4)
  } else {
    if (split == 4) VG_GDN_PF(4, 2)
    else if (split == 2) VG_GDN_PF(2, 2)
    else VG_GDN_PF(1, 2)
  }
#undef VG_GDN_PF
  if (split > 1)
    launch_pdl(gdn_out_norm_kernel<128>, dim3((unsigned)(((size_t)tn * nv + 7) / 8)), dim3(256), 0, st, (const float*)o_scratch, pj, ldp,
               off_z, norm_w, t0, tn, o16, nv, eps);
  return (int)cudaGetLastError();
}

// Gated output norm over fp32 raw outputs [t][nv][vd] (shared with the chunked prefill in gdn_chunk.cu).
int vg_gdn_out_norm_launch(const float* o_raw, const void* proj, int ldp, int off_z, const float* norm_w, int t0, int tn,
                           void* out_f16, int nv, int vd, float eps, cudaStream_t st) {
  if (vd != 128) return -3;
  return (int)launch_pdl(gdn_out_norm_kernel<128>, dim3((unsigned)(((size_t)tn * nv + 7) / 8)), dim3(256), 0, st, o_raw,
                         static_cast<const __nv_bfloat16*>(proj), ldp, off_z, norm_w, t0, tn, static_cast<__half*>(out_f16), nv, eps);
}

VG_TRACE_SETTER(vg_trace_set_gdn)

// GQA attention over the slotted KV cache: flash-decoding style split-K kernel + fixed-order merge.
//
// One CTA serves (column, kv head, query sub-group, split). Its 8 warps walk the split's keys in a
// fixed interleave (warp w takes keys k0+w, k0+w+8, ...), each lane owning hd/32 dims, with an online
// softmax per query head in fp32; the warps' (m, l, acc) are merged in warp order. The number of
// splits is a pure function of the column's own key count, ns = clamp(len/64, 1, 32), so a column is
// computed the same way whether it runs alone or beside 15 others (reference:
// kernels/gpu_batch.cu:1443-1477, :1491-1606, :2151-2186). Keys at or beyond `base[col]` are addressed
// through a per-column row list (tree / forest verify); before it, key t is cache row t.
// The merge kernel combines the splits in index order, normalises, applies the sigmoid output gate
// and emits the f16 input of o_proj. Prefill uses the same kernel with one split per column and the
// gate applied directly (it is outside the batch-invariance contract).
//
// The partial buffer (m, l, acc[hd]) per (column, head, split) is scratch memory owned by the caller.
#include <cstdio>
#include <mutex>

#include "common.cuh"
#include "api.h"
#include "attention_static.h"

namespace {
using namespace vg;

constexpr int NW = 8;   // warps per CTA

// Splits of a column: one per 64 keys, at most 32 and never more than the launch grid (and the partial buffer)
// provides, so a caller that passes a smaller `ns_grid` gets fewer, longer splits instead of dropped keys.
__device__ __forceinline__ int splits_for(int len, int ns_grid) {
  int ns = len / 64;
  ns = ns < 1 ? 1 : (ns > 32 ? 32 : ns);
  return ns > ns_grid ? ns_grid : ns;
}

// One lane's DPL consecutive bf16 values of a cache row, fetched with a single vector load.
template <int DPL> struct RowVec;
template <> struct RowVec<8> { using T = uint4; };
template <> struct RowVec<4> { using T = uint2; };
template <> struct RowVec<2> { using T = uint32_t; };
template <> struct RowVec<1> { using T = unsigned short; };
// DPL 4-bit codes of one lane (DPL / 2 bytes).
template <int DPL> struct CodeVec;
template <> struct CodeVec<8> { using T = uint32_t; };
template <> struct CodeVec<4> { using T = unsigned short; };
template <> struct CodeVec<2> { using T = uint8_t; };
template <> struct CodeVec<1> { using T = uint8_t; };
template <int DPL>
__device__ __forceinline__ void unpack_row(const typename RowVec<DPL>::T& raw, float* f) {
  const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
  for (int i = 0; i < DPL; ++i) f[i] = __bfloat162float(h[i]);
}

// Q4: the cache holds 4-bit codes (two per byte, value + 8, symmetric +-7) with one f16 scale per 16 values;
// kc / vc then point at the code bytes and ks / vs at the scales (reference: kernels/gpu_batch.cu:729-802, :1606).
template <int HD, int GT, bool Q4>
__global__ void __launch_bounds__(NW * 32) attn_split_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kc, const __nv_bfloat16* __restrict__ vc,
    const __half* __restrict__ ks, const __half* __restrict__ vs, const int* __restrict__ lens, const int* __restrict__ slots, const int* __restrict__ base,
    const int* __restrict__ path, int path_ld, float* __restrict__ part, int nh, int nkv, int max_seq, int ns_grid,
    float scale, int direct, const __nv_bfloat16* __restrict__ gate, int ld_gate, int gate_off, __half* __restrict__ out) {
  pdl_trigger();
  pdl_wait();
  constexpr int DPL = HD / 32;              // dims per lane
  const int col = blockIdx.x;
  const int G = nh / nkv;
  const int nsub = G / GT;
  const int kvh = blockIdx.y / nsub, sub = blockIdx.y % nsub;
  const int split = blockIdx.z;
  const int len = lens[col];
  const int ns = direct ? 1 : splits_for(len, ns_grid);
  if (split >= ns) return;
  const int chunk = (len + ns - 1) / ns;
  const int k0 = split * chunk;
  const int k1 = min(len, k0 + chunk);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slot = slots[col];
  const int kbase = base ? base[col] : len;
  const int h0 = kvh * G + sub * GT;        // first query head of this CTA

  float qf[GT][DPL];
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    const __nv_bfloat16* qp = q + ((size_t)col * nh + h0 + g) * HD + lane * DPL;
#pragma unroll
    for (int i = 0; i < DPL; ++i) qf[g][i] = __bfloat162float(qp[i]) * scale;
  }
  float m[GT], l[GT], acc[GT][DPL];
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[g][i] = 0.f;
  }
  const size_t head_rows = ((size_t)slot * nkv + kvh) * (size_t)max_seq;
  const __nv_bfloat16* kslot = kc + head_rows * HD;
  const __nv_bfloat16* vslot = vc + head_rows * HD;
  // 4-bit cache: DPL / 2 code bytes per lane and the scale of the 16-value block the lane's dims fall into
  using Codes = typename CodeVec<DPL>::T;
  const uint8_t* kq = reinterpret_cast<const uint8_t*>(kc) + head_rows * (HD / 2);
  const uint8_t* vq = reinterpret_cast<const uint8_t*>(vc) + head_rows * (HD / 2);
  const __half* ksc = Q4 ? ks + head_rows * (HD / 16) : nullptr;
  const __half* vsc = Q4 ? vs + head_rows * (HD / 16) : nullptr;

  // Keys of this warp in batches of U: all loads of a batch are issued before its first dot product, so a
  // warp keeps U rows of K and V in flight; the keys are still folded in in ascending order.
  constexpr int U = 4;
  using Raw = typename RowVec<DPL>::T;
  for (int tb = k0 + warp; tb < k1; tb += NW * U) {
    Raw kraw[U], vraw[U];
    Codes kcd[U], vcd[U];
    __half ksv[U], vsv[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int t = tb + u * NW;
      if (t < k1) {
        const int row = t < kbase ? t : path[(size_t)col * path_ld + (t - kbase)];
        if (Q4) {
          kcd[u] = *reinterpret_cast<const Codes*>(kq + (size_t)row * (HD / 2) + lane * (DPL / 2));
          vcd[u] = *reinterpret_cast<const Codes*>(vq + (size_t)row * (HD / 2) + lane * (DPL / 2));
          ksv[u] = ksc[(size_t)row * (HD / 16) + (lane * DPL) / 16];
          vsv[u] = vsc[(size_t)row * (HD / 16) + (lane * DPL) / 16];
        } else {
          kraw[u] = *reinterpret_cast<const Raw*>(kslot + (size_t)row * HD + lane * DPL);
          vraw[u] = *reinterpret_cast<const Raw*>(vslot + (size_t)row * HD + lane * DPL);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (tb + u * NW >= k1) break;
      float kf[DPL], vf[DPL];
      if (Q4) {
        const uint8_t* kb = reinterpret_cast<const uint8_t*>(&kcd[u]);
        const uint8_t* vb = reinterpret_cast<const uint8_t*>(&vcd[u]);
        const float sk = __half2float(ksv[u]), sv = __half2float(vsv[u]);
#pragma unroll
        for (int i = 0; i < DPL / 2; ++i) {
          kf[2 * i] = (float)((int)(kb[i] & 15) - 8) * sk; kf[2 * i + 1] = (float)((int)(kb[i] >> 4) - 8) * sk;
          vf[2 * i] = (float)((int)(vb[i] & 15) - 8) * sv; vf[2 * i + 1] = (float)((int)(vb[i] >> 4) - 8) * sv;
        }
      } else {
        unpack_row<DPL>(kraw[u], kf);
        unpack_row<DPL>(vraw[u], vf);
      }
#pragma unroll
      for (int g = 0; g < GT; ++g) {
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < DPL; ++i) s = fmaf(qf[g][i], kf[i], s);
        s = warp_sum(s);
        const float mn = fmaxf(m[g], s);
        const float corr = __expf(m[g] - mn);
        const float p = __expf(s - mn);
        l[g] = l[g] * corr + p;
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[g][i] = fmaf(p, vf[i], acc[g][i] * corr);
        m[g] = mn;
      }
    }
  }

  // merge the warps in warp order through shared memory
  __shared__ float sm_m[NW][GT], sm_l[NW][GT];
  __shared__ float sm_acc[NW][GT][HD];
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    if (lane == 0) { sm_m[warp][g] = m[g]; sm_l[warp][g] = l[g]; }
#pragma unroll
    for (int i = 0; i < DPL; ++i) sm_acc[warp][g][lane * DPL + i] = acc[g][i];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < GT * HD; idx += blockDim.x) {
    const int g = idx / HD, d = idx % HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < NW; ++w) M = fmaxf(M, sm_m[w][g]);
    float L = 0.f, A = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      const float e = sm_m[w][g] == -INFINITY ? 0.f : __expf(sm_m[w][g] - M);
      L += sm_l[w][g] * e;
      A += sm_acc[w][g][d] * e;
    }
    const int head = h0 + g;
    if (direct) {
      float o = L > 0.f ? A / L : 0.f;
      if (gate) o *= sigmoidf(__bfloat162float(gate[(size_t)col * ld_gate + (size_t)head * gate_off * 2 + gate_off + d]));
      out[((size_t)col * nh + head) * HD + d] = f32_to_f16_sat(o);
    } else {
      float* pp = part + (((size_t)col * nh + head) * ns_grid + split) * (HD + 2);
      if (d == 0) { pp[0] = M; pp[1] = L; }
      pp[2 + d] = A;
    }
  }
}

template <int HD>
__global__ void attn_merge_kernel(const float* __restrict__ part, const int* __restrict__ lens, int nh, int ns_grid,
                                  const __nv_bfloat16* __restrict__ gate, int ld_gate, __half* __restrict__ out) {
  pdl_trigger();
  pdl_wait();
  const int col = blockIdx.x, head = blockIdx.y, d = threadIdx.x;
  const int ns = splits_for(lens[col], ns_grid);
  const float* pp = part + ((size_t)col * nh + head) * ns_grid * (HD + 2);
  // every split's three values are fetched before the first is used (the loads are independent: one L2 latency, not
  // one per split); the sums still run over the splits in index order
  float ms[32], ls[32], as[32];
#pragma unroll
  for (int s = 0; s < 32; ++s) {
    const bool on = s < ns;
    ms[s] = on ? pp[(size_t)s * (HD + 2)] : -INFINITY;
    ls[s] = on ? pp[(size_t)s * (HD + 2) + 1] : 0.f;
    as[s] = on ? pp[(size_t)s * (HD + 2) + 2 + d] : 0.f;
  }
  float M = -INFINITY;
#pragma unroll
  for (int s = 0; s < 32; ++s) M = fmaxf(M, ms[s]);
  float L = 0.f, A = 0.f;
#pragma unroll
  for (int s = 0; s < 32; ++s) {
    if (s < ns) {
      const float e = ms[s] == -INFINITY ? 0.f : __expf(ms[s] - M);
      L += ls[s] * e;
      A += as[s] * e;
    }
  }
  float o = L > 0.f ? A / L : 0.f;
  // gate layout inside the fused qkv row: head h occupies [h*2hd, h*2hd+hd) = q, [.. + hd, .. + 2hd) = gate
  if (gate) o *= sigmoidf(__bfloat162float(gate[(size_t)col * ld_gate + (size_t)head * 2 * HD + HD + d]));
  out[((size_t)col * nh + head) * HD + d] = f32_to_f16_sat(o);
}

template <int HD, int GT>
int launch_split(const void* q, const void* kc, const void* vc, const void* ks, const void* vs, const int* lens, const int* slots, const int* base,
                 const int* path, int path_ld, float* part, int N, int nh, int nkv, int max_seq, int ns_grid, int direct,
                 const void* gate, int ld_gate, void* out, cudaStream_t st) {
  const int G = nh / nkv;
  dim3 grid(N, nkv * (G / GT), direct ? 1 : ns_grid);
  if (ks)
    launch_pdl(attn_split_kernel<HD, GT, true>, dim3(grid), dim3(NW * 32), 0, st, static_cast<const __nv_bfloat16*>(q),
               static_cast<const __nv_bfloat16*>(kc), static_cast<const __nv_bfloat16*>(vc), static_cast<const __half*>(ks),
               static_cast<const __half*>(vs), lens, slots, base, path, path_ld, part, nh, nkv, max_seq, ns_grid,
               rsqrtf((float)HD), direct, static_cast<const __nv_bfloat16*>(gate), ld_gate, HD, static_cast<__half*>(out));
  else
    launch_pdl(attn_split_kernel<HD, GT, false>, dim3(grid), dim3(NW * 32), 0, st, static_cast<const __nv_bfloat16*>(q),
               static_cast<const __nv_bfloat16*>(kc), static_cast<const __nv_bfloat16*>(vc), (const __half*)nullptr,
               (const __half*)nullptr, lens, slots, base, path, path_ld, part, nh, nkv, max_seq, ns_grid,
               rsqrtf((float)HD), direct, static_cast<const __nv_bfloat16*>(gate), ld_gate, HD, static_cast<__half*>(out));
  return (int)cudaGetLastError();
}

template <int HD>
int dispatch_gt(int G, const void* q, const void* kc, const void* vc, const void* ks, const void* vs, const int* lens, const int* slots, const int* base,
                const int* path, int path_ld, float* part, int N, int nh, int nkv, int max_seq, int ns_grid, int direct,
                const void* gate, int ld_gate, void* out, cudaStream_t st) {
#define VG_ARGS q, kc, vc, ks, vs, lens, slots, base, path, path_ld, part, N, nh, nkv, max_seq, ns_grid, direct, gate, ld_gate, out, st
  if (HD == 256) {
    if (G % 4 == 0) return launch_split<HD, 4>(VG_ARGS);
    if (G % 3 == 0) return launch_split<HD, 3>(VG_ARGS);
    if (G % 2 == 0) return launch_split<HD, 2>(VG_ARGS);
    return launch_split<HD, 1>(VG_ARGS);
  }
  if (G % 4 == 0) return launch_split<HD, 4>(VG_ARGS);
  if (G % 3 == 0) return launch_split<HD, 3>(VG_ARGS);
  if (G % 2 == 0) return launch_split<HD, 2>(VG_ARGS);
  return launch_split<HD, 1>(VG_ARGS);
#undef VG_ARGS
}

}  // namespace

// q [N, nh, hd] bf16; kc/vc [slots, nkv, max_seq, hd] bf16; lens[N] keys per column; slots[N];
// base[N]/path[N, path_ld] optional row indirection; part: scratch of vg_attn_scratch_floats() floats;
// gate: fused qkv buffer (bf16, row stride ld_gate) or null; out [N, nh*hd] f16.
namespace {
int attn_decode_impl(const void* q, const void* kc, const void* vc, const void* ks, const void* vs, const int* lens,
                     const int* slots, const int* base, const int* path, int path_ld, float* part, int N, int nh, int nkv,
                     int hd, int max_seq, int ns_grid, int direct, const void* gate, int ld_gate, void* out, cudaStream_t st) {
  if (N <= 0) return 0;
  if (nh % nkv || (!direct && ns_grid < 1)) return -2;
  const int G = nh / nkv;
  int rc;
  switch (hd) {
    case 64: rc = dispatch_gt<64>(G, q, kc, vc, ks, vs, lens, slots, base, path, path_ld, part, N, nh, nkv, max_seq, ns_grid, direct, gate, ld_gate, out, st); break;
    case 128: rc = dispatch_gt<128>(G, q, kc, vc, ks, vs, lens, slots, base, path, path_ld, part, N, nh, nkv, max_seq, ns_grid, direct, gate, ld_gate, out, st); break;
    case 256: rc = dispatch_gt<256>(G, q, kc, vc, ks, vs, lens, slots, base, path, path_ld, part, N, nh, nkv, max_seq, ns_grid, direct, gate, ld_gate, out, st); break;
    default: return -3;
  }
  if (rc || direct) return rc;
  dim3 grid(N, nh);
  switch (hd) {
    case 64: launch_pdl(attn_merge_kernel<64>, dim3(grid), dim3(64), 0, st, part, lens, nh, ns_grid, static_cast<const __nv_bfloat16*>(gate), ld_gate, static_cast<__half*>(out)); break;
    case 128: launch_pdl(attn_merge_kernel<128>, dim3(grid), dim3(128), 0, st, part, lens, nh, ns_grid, static_cast<const __nv_bfloat16*>(gate), ld_gate, static_cast<__half*>(out)); break;
    case 256: launch_pdl(attn_merge_kernel<256>, dim3(grid), dim3(256), 0, st, part, lens, nh, ns_grid, static_cast<const __nv_bfloat16*>(gate), ld_gate, static_cast<__half*>(out)); break;
  }
  return (int)cudaGetLastError();
}
}  // namespace

// Merge of split partials (shared with the tensor-core split kernel in attention_decode_tc.cu).
int vg_attn_merge_launch(const float* part, const int* lens, int N, int nh, int hd, int ns_grid, const void* gate, int ld_gate,
                         void* out, cudaStream_t st) {
  dim3 grid(N, nh);
  switch (hd) {
    case 64: launch_pdl(attn_merge_kernel<64>, dim3(grid), dim3(64), 0, st, part, lens, nh, ns_grid, static_cast<const __nv_bfloat16*>(gate), ld_gate, static_cast<__half*>(out)); break;
    case 128: launch_pdl(attn_merge_kernel<128>, dim3(grid), dim3(128), 0, st, part, lens, nh, ns_grid, static_cast<const __nv_bfloat16*>(gate), ld_gate, static_cast<__half*>(out)); break;
    case 256: launch_pdl(attn_merge_kernel<256>, dim3(grid), dim3(256), 0, st, part, lens, nh, ns_grid, static_cast<const __nv_bfloat16*>(gate), ld_gate, static_cast<__half*>(out)); break;
    default: return -3;
  }
  return (int)cudaGetLastError();
}

// q [N, nh, hd] bf16; kc/vc [slots, nkv, max_seq, hd] bf16; lens[N] keys per column; slots[N];
// base[N]/path[N, path_ld] optional row indirection; part: scratch of vg_attn_scratch_floats() floats;
// gate: fused qkv buffer (bf16, row stride ld_gate) or null; out [N, nh*hd] f16.
extern "C" int vg_attn_decode(const void* q, const void* kc, const void* vc, const int* lens, const int* slots,
                              const int* base, const int* path, int path_ld, float* part, int N, int nh, int nkv, int hd,
                              int max_seq, int ns_grid, int direct, const void* gate, int ld_gate, void* out,
                              cudaStream_t st) {
  return attn_decode_impl(q, kc, vc, nullptr, nullptr, lens, slots, base, path, path_ld, part, N, nh, nkv, hd, max_seq, ns_grid,
                          direct, gate, ld_gate, out, st);
}

// Same over the 4-bit cache: kq/vq [slots, nkv, max_seq, hd/2] code bytes, ks/vs [slots, nkv, max_seq, hd/16] f16 scales.
extern "C" int vg_attn_decode_q4(const void* q, const void* kq, const void* vq, const void* ks, const void* vs, const int* lens,
                                 const int* slots, const int* base, const int* path, int path_ld, float* part, int N, int nh,
                                 int nkv, int hd, int max_seq, int ns_grid, int direct, const void* gate, int ld_gate, void* out,
                                 cudaStream_t st) {
  if (!ks || !vs) return -2;
  return attn_decode_impl(q, kq, vq, ks, vs, lens, slots, base, path, path_ld, part, N, nh, nkv, hd, max_seq, ns_grid, direct, gate,
                          ld_gate, out, st);
}

extern "C" long long vg_attn_scratch_floats(int N, int nh, int hd, int ns_grid) {
  return (long long)N * nh * ns_grid * (hd + 2);
}

// ------------------------------------------------------------------ allocation-free variant
namespace {
// Split-K partials for vg_attn_decode_static: lives in the library image, one copy per GPU.
static __device__ __align__(256) float g_attn_static_scratch[VG_ATTN_STATIC_MAX_FLOATS];

constexpr int kMaxDevices = 64;
float* g_static_ptr[kMaxDevices] = {};
std::mutex g_static_mu;

// Device address of the static array on the current device (the host-side symbol is only a stand-in and
// must never be handed to a kernel). Looked up once per device.
int static_scratch_ptr(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return -2;
  std::lock_guard<std::mutex> lk(g_static_mu);
  if (!g_static_ptr[dev]) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_attn_static_scratch);
    if (e != cudaSuccess) return (int)e;
    g_static_ptr[dev] = p;
  }
  *out = g_static_ptr[dev];
  return 0;
}
}  // namespace

extern "C" int vg_attn_decode_static(const void* q, const void* kc, const void* vc, const int* lens, const int* slots,
                                     const int* base, const int* path, int path_ld, int N, int nh, int nkv, int hd,
                                     int max_seq, int ns_grid, int direct, const void* gate, int ld_gate, void* out,
                                     cudaStream_t stream) {
  const long long need = direct ? 0 : vg_attn_scratch_floats(N, nh, hd, ns_grid);
  if (need > VG_ATTN_STATIC_MAX_FLOATS) {
    fprintf(stderr,
            "vg_attn_decode_static: %lld floats of split-K scratch needed (N=%d heads=%d head_dim=%d splits=%d) but the "
            "built-in buffer holds %lld; use vg_attn_decode with a caller-provided buffer\n",
            need, N, nh, hd, ns_grid, (long long)VG_ATTN_STATIC_MAX_FLOATS);
    return VG_ERR_STATIC_SCRATCH;
  }
  float* part = nullptr;
  const int rc = static_scratch_ptr(&part);
  if (rc) return rc;
  return vg_attn_decode(q, kc, vc, lens, slots, base, path, path_ld, part, N, nh, nkv, hd, max_seq, ns_grid, direct, gate,
                        ld_gate, out, stream);
}

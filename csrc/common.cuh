// Shared device helpers for the sm_100a kernels: PTX wrappers for mbarrier, bulk/tensor TMA copies,
// tcgen05 (TMEM allocation, UMMA issue, commit, TMEM loads), cluster barriers and DSMEM access, plus
// small numeric helpers. Every wait is bounded: on expiry the caller records an error code in a
// device status word and unwinds, so a lost signal can never hang the GPU.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdlib.h>
#include <utility>

#define VG_DEVINL __device__ __forceinline__

// Error codes written to the status word passed to kernels (0 = ok).
enum VgErr : int {
  VG_OK = 0,
  VG_ERR_TMA_WAIT = 1,      // consumer waited too long for a TMA stage
  VG_ERR_EMPTY_WAIT = 2,    // producer waited too long for a free stage
  VG_ERR_MMA_WAIT = 3,      // epilogue waited too long for the accumulator
  VG_ERR_PEER_WAIT = 4,     // a peer rank's flag did not arrive in time
  VG_ERR_BAD_ARG = 5,
  VG_ERR_DEQ_WAIT = 6,
  VG_ERR_GRID_WAIT = 7,     // CTAs of one grid waited too long for each other
};

namespace vg {

VG_DEVINL uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

VG_DEVINL bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .pred P;\n\t.reg .b32 R;\n\t"
      "elect.sync R|P, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t}\n"
      : "=r"(pred));
  return pred != 0;
}

// ------------------------------------------------------------------ mbarrier
VG_DEVINL void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
VG_DEVINL void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
VG_DEVINL void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

VG_DEVINL void mbar_arrive(uint64_t* bar) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(smem_u32(bar)) : "memory");
}
VG_DEVINL void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
VG_DEVINL bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t}\n"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
VG_DEVINL uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: gives up after `budget_ns` of wall time (default 200 ms). Returns false when the budget
// ran out (the caller reports and unwinds).
VG_DEVINL bool mbar_wait(uint64_t* bar, uint32_t parity, uint64_t budget_ns = 200ull * 1000 * 1000) {
  for (int i = 0; i < 64; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  const uint64_t t0 = global_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (global_ns() - t0 > budget_ns) return false;
  }
}

// ------------------------------------------------------------------ TMA
// 1-D bulk copy global -> shared, completion counted in bytes on an mbarrier. Addresses and size
// must be multiples of 16 bytes.
VG_DEVINL void tma_bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// 2-D tiled tensor copy global -> shared (no multicast). c0 is the innermost coordinate and must make
// c0 * elem_size a multiple of 16 bytes.
VG_DEVINL void tma_tensor2d_g2s(void* smem_dst, const void* tmap, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_u32(smem_dst)),
      "l"(tmap), "r"(c0), "r"(c1), "r"(smem_u32(bar))
      : "memory");
}
VG_DEVINL void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ------------------------------------------------------------------ tcgen05 / TMEM
VG_DEVINL void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols)
               : "memory");
}
VG_DEVINL void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
VG_DEVINL void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
VG_DEVINL void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
VG_DEVINL void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptor for a K-major operand tile stored with the 128-byte swizzle:
// rows are 128 bytes (64 x 16-bit), groups of 8 rows are 1024 bytes apart.
VG_DEVINL uint64_t umma_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);        // start address, bits [0,14)
  d |= (uint64_t)1 << 16;                             // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;                   // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                             // descriptor version for sm_100
  d |= (uint64_t)2 << 61;                             // layout type: SWIZZLE_128B
  return d;
}
// Instruction descriptor for kind::f16 with fp32 accumulation, both operands K-major.
// fmt: 0 = f16, 1 = bf16.
VG_DEVINL constexpr uint32_t umma_idesc_f16(int m, int n, int afmt, int bfmt) {
  return (1u << 4) | ((uint32_t)afmt << 7) | ((uint32_t)bfmt << 10) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}
VG_DEVINL void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Make an mbarrier track completion of all tcgen05 operations issued so far by this thread.
VG_DEVINL void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
VG_DEVINL void tmem_ld8(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
VG_DEVINL void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ------------------------------------------------------------------ clusters / DSMEM
VG_DEVINL uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
VG_DEVINL void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Split form for "every CTA of the cluster has started": arrive at kernel entry, wait just before the first store
// into a peer's shared memory (by then the wait returns at once).
VG_DEVINL void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory"); }
VG_DEVINL void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
VG_DEVINL uint32_t dsmem_map(uint32_t local_addr, uint32_t cta_rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(cta_rank));
  return r;
}
VG_DEVINL float dsmem_ld_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}

VG_DEVINL void dsmem_st_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

// ------------------------------------------------------------------ peer-memory flags
constexpr int MAX_RANKS = 8;
constexpr int MAX_CTAS = 64;
constexpr int FLAG_STRIDE = 32;      // uint32 per flag line (128 bytes)

VG_DEVINL void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
VG_DEVINL uint32_t ld_acquire_gpu(const unsigned int* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
VG_DEVINL uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Wait until *p has reached epoch e (wrap-safe). False when the budget ran out.
VG_DEVINL bool wait_flag(const uint32_t* p, uint32_t e, uint64_t budget_ns) {
  for (int i = 0; i < 256; ++i)
    if ((int32_t)(ld_acquire_sys(p) - e) >= 0) return true;
  const uint64_t t0 = global_ns();
  for (;;) {
    for (int i = 0; i < 64; ++i)
      if ((int32_t)(ld_acquire_sys(p) - e) >= 0) return true;
    if (global_ns() - t0 > budget_ns) return false;
  }
}

// NVLS (NVLink-switch multicast) accesses on a multicast address: the store reaches every rank's copy of the word;
// the load returns the sum over all ranks' copies of four consecutive fp32 values, added inside the switch.
VG_DEVINL void multimem_st_u32(void* mc_addr, uint32_t v) {
  asm volatile("multimem.st.relaxed.sys.global.u32 [%0], %1;" ::"l"(mc_addr), "r"(v) : "memory");
}
VG_DEVINL float4 multimem_ld_reduce_f32x4(const void* mc_addr) {
  float4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w) : "l"(mc_addr) : "memory");
  return r;
}

// Eight bf16 values: sum over all ranks' copies (fp32 accumulation inside the switch) / store to all ranks' copies.
VG_DEVINL uint4 multimem_ld_reduce_bf16x8(const void* mc_addr) {
  uint4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(mc_addr) : "memory");
  return r;
}
VG_DEVINL void multimem_st_bf16x8(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w) : "memory");
}

VG_DEVINL size_t flag_index(int set, int src, int cta) {
  return ((size_t)(set * MAX_RANKS + src) * MAX_CTAS + cta) * FLAG_STRIDE;
}


// ------------------------------------------------------------------ numerics
VG_DEVINL float bf16_to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
VG_DEVINL float silu(float x) { return x / (1.0f + __expf(-x)); }
VG_DEVINL float sigmoidf(float x) { return 1.0f / (1.0f + __expf(-x)); }

// f32 -> f16 with saturation to the largest finite value (GEMM inputs are f16).
VG_DEVINL __half f32_to_f16_sat(float v) {
  v = fminf(fmaxf(v, -65504.0f), 65504.0f);
  return __float2half_rn(v);
}

VG_DEVINL float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
VG_DEVINL float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum with a fixed reduction tree (deterministic). `red` holds >= 32 floats.
VG_DEVINL float block_sum(float v, float* red) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.0f;
  t = warp_sum(t);
  return t;
}

// ---------------------------------------------------------------- device timeline (builds with -DVG_TRACE only)
// trace(code) appends (global nanosecond timer, code, blockIdx.x) to a host-provided buffer; buffer word 0 is
// the record counter. Each translation unit has its own pointer, set through the setter VG_TRACE_SETTER
// defines. Without -DVG_TRACE both compile to nothing.
#ifdef VG_TRACE
static __device__ unsigned long long* vg_trace_buf = nullptr;
static __device__ unsigned int vg_trace_cap = 0;
VG_DEVINL void trace(int code) {
  unsigned long long* b = vg_trace_buf;
  if (!b) return;
  const unsigned i = atomicAdd(reinterpret_cast<unsigned int*>(b), 1u);
  if (i < vg_trace_cap) {
    b[1 + 2 * i] = global_ns();
    b[2 + 2 * i] = ((unsigned long long)blockIdx.x << 32) | ((unsigned long long)blockIdx.z << 16) | (unsigned)code;
  }
}
#define VG_TRACE_SETTER(fn)                                            \
  extern "C" int fn(void* buf, unsigned cap) {                         \
    cudaError_t e = cudaMemcpyToSymbol(vg_trace_buf, &buf, sizeof(buf)); \
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(vg_trace_cap, &cap, sizeof(cap)); \
    return (int)e;                                                     \
  }
#else
VG_DEVINL void trace(int) {}
#define VG_TRACE_SETTER(fn) \
  extern "C" int fn(void*, unsigned) { return -1; }
#endif

// ---------------------------------------------------------------- programmatic dependent launch
// A kernel launched through launch_pdl may start while its predecessor in the stream is still running.
// Every such kernel executes pdl_wait() before it reads anything a predecessor wrote or writes anything a
// predecessor may still read (it returns at once when there is no programmatic dependency), so completion of
// a kernel implies completion of all earlier ones. pdl_trigger() lets the successor be scheduled as soon as
// every CTA of this grid has started; work that does not depend on the predecessor (streaming weights into
// shared memory, barrier and TMEM setup) then overlaps the predecessor's tail.
VG_DEVINL void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
VG_DEVINL void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline bool pdl_on() {
  static const bool on = [] { const char* e = getenv("VELO_NO_PDL"); return !(e && e[0] == '1'); }();
  return on;
}
// `cluster_x` > 1 launches thread-block clusters of that many CTAs along x (grid.x must be a multiple).
template <typename... KA, typename... A>
inline cudaError_t launch_pdl_cluster(void (*kernel)(KA...), dim3 grid, dim3 block, unsigned cluster_x, size_t smem,
                                      cudaStream_t st, A&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (cluster_x > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = cluster_x;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  if (pdl_on()) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<A>(args)...);
}
template <typename... KA, typename... A>
inline cudaError_t launch_pdl(void (*kernel)(KA...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, A&&... args) {
  return launch_pdl_cluster(kernel, grid, block, 1u, smem, st, std::forward<A>(args)...);
}

}  // namespace vg

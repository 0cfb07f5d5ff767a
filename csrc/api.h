// C ABI of the velogb10_b200 kernel library (loaded from Python through ctypes).
// All pointers are device pointers unless stated otherwise; every function enqueues work on `stream`
// and returns 0 on success (a negative value for a rejected argument, a positive cudaError_t otherwise).
#pragma once
#include <cuda_runtime.h>

// weight formats
#define VG_WF_NVFP4 0   // e2m1 codes + e4m3 scale per 16 along K
#define VG_WF_FP8 1     // e4m3 codes, fp32 scale per row
#define VG_WF_F16 2     // tile-major f16 (tensor-core GEMM input made from bf16 weights)
#define VG_WF_BF16 3    // canonical row-major bf16 (CUDA-core GEMV, embedding)

#ifdef __cplusplus
extern "C" {
#endif

// Peer-memory communication context (one per rank; data[q] is rank q's symmetric arena mapped here).
typedef struct VgCommCtx {
  int rank, world;
  unsigned char* data[8];
  unsigned long long flags_off, slots_off, slot_bytes, result_off, result_bytes;
  unsigned int* epoch;       // device-resident epoch counter of this rank
  unsigned int* done_ctr;    // CTA completion counter
  int* status;               // error status word (0 = ok)
  unsigned long long timeout_ns;
  unsigned long long agbuf_off, agbuf_bytes;  // gather landing zone of the fused all-gather + GEMM (f16 rows)
  unsigned long long agflags_off;  // [2 sets][VG_AG_MAX_TILES] epoch per 128-row tile of the landing zone
  unsigned long long rsflags_off;  // [2 sets][8 ranks][VG_RS_MAX_TILES] per-tile epochs of the fused GEMM + reduce-scatter
  // NVLink-switch multicast (NVLS) view of the same arena: one address that reaches every rank's copy. Stores to it
  // (multimem.st) land on all ranks; multimem.ld_reduce returns the sum of all ranks' copies, added inside the
  // switch. Null when the arena has no multicast binding (then only the peer-pointer paths run).
  unsigned char* mc;
  unsigned long long mm_off, mm_slot_bytes;   // [2 sets][mm_slot_bytes] fp32 partial rows, written locally by their owner
  unsigned long long mmflags_off;             // [2 sets][64 tiles][8 ranks] word = epoch of that rank's rows of the tile
  unsigned int* mm_ctr;                       // (spare control word)
} VgCommCtx;
#define VG_RS_MAX_TILES 4096
#define VG_AG_MAX_TILES 256
#define VG_ARGMAX_MAX_COLS 64     // columns vg_comm_argmax_merge accepts (size of the callers' pair buffers)

// Optional epilogue of the decode-width GEMM that produces the GatedDeltaNet input projection: rows below
// conv_dim are conv channels, and the thread that owns a row runs the depthwise causal conv + SiLU for every
// column and updates the rolling conv state, so no separate conv kernel is needed
// (column bookkeeping as in vg_gdn_conv).
typedef struct VgConvEpi {
  float* state;              // [slot][conv_dim][ck]
  const float* w;            // [conv_dim][ck]
  const int* in_slot;
  const int* parent;
  const int* out_slot;
  float* out;                // [N][conv_dim] fp32
  int conv_dim, ck;
} VgConvEpi;

int vg_gemm_tc(const void* wt, const float* row_scale, const void* x_f16, int x_rows, int ldx, void* out, int out_f32,
               int M, int K, int N, int ldo, int wfmt, int splitk, int* err, const VgCommCtx* ar_ctx, int rs_rows, int ag,
               cudaStream_t stream);
// Second half of the fused GEMM + reduce-scatter (prefill widths): vg_gemm_tc(..., ar_ctx, rs_rows > 0) made every
// rank push each partial output tile straight into the receive slot of the rank that owns the tile's token rows
// (rows [p * rs_rows, (p + 1) * rs_rows) belong to rank p) and publish a per-tile epoch. This kernel waits for the
// tiles of its own rows from every rank, sums them in rank order, broadcasts the bf16 result and assembles
// out [n, M] on every rank.
// Fused all-gather + GEMM (column-parallel layer whose input is sharded by token rows): every rank pushes its shard
// (rows [row0, row0 + rows), whole 128-row tiles) into every rank's landing zone and publishes one epoch word per
// tile; vg_gemm_tc(..., ag = 1) then reads the landing zone and holds the TMA loads of a token tile until that
// tile's word has arrived, so the GEMM starts on the local rows while the others are still in flight.
int vg_comm_ag_push(const VgCommCtx* ctx, const void* x_f16, int row0, int rows, int K, cudaStream_t stream);
int vg_comm_gemm_rs_finish(const VgCommCtx* ctx, void* out_bf16, int n, int M, int rs_rows, cudaStream_t stream);
int vg_act_quant_fp4(const void* x_f16, int ldx, int N, int K, void* bq, int ldb, void* sfb, float* g0, cudaStream_t stream);
int vg_swiglu_fp4(const void* gu, int ld, int N, int I, void* bq, int ldb, void* sfb, float* g0, void* out16,
                  cudaStream_t stream);
int vg_add_rmsnorm_fp4(void* res, const void* delta, const float* w, int N, int h, float eps, int plus_one, int ld_res,
                       int ld_delta, void* bq, int ldb, void* sfb, float* g0, void* out16, cudaStream_t stream);
int vg_gemm_fp4(const void* wt, const float* row_scale, const void* bq, int ldb, const void* sfb, const float* g0, void* out,
                int out_f32, int M, int K, int N, int ldo, int splitk, int* err, const VgCommCtx* ar_ctx, int ar_push_only,
                const VgConvEpi* conv, cudaStream_t stream);
// Residual add + RMSNorm + FP4 quantisation whose `delta` is the tensor-parallel sum of the partial rows a
// preceding vg_gemm_fp4(..., ar_push_only = 1) pushed into every rank's receive slots: waits for each
// rank's tile flags (bounded), adds the partials in rank order, then proceeds as vg_add_rmsnorm_fp4.
// mode 1: (value, epoch) pairs in the per-rank receive slots (ar_push_only = 1). mode 2: in-switch reduction: the
// partial rows were written by vg_gemm_fp4(..., ar_push_only = 2) into each rank's own multimem slot; the kernel waits
// for every rank's epoch word and reads each element once with multimem.ld_reduce (needs ctx->mc).
int vg_add_rmsnorm_fp4_ar(void* res, const float* w, int N, int h, float eps, int plus_one, int ld_res, void* bq, int ldb,
                          void* sfb, float* g0, void* out16, const VgCommCtx* ctx, int mode, cudaStream_t stream);
int vg_gemm_fp4_grouped(const void* wt, const float* row_scale, const void* bq, int ldb, int b_rows, const void* sfb,
                        const float* g0, void* out, int out_f32, int M, int K, int ldo, int n_items, const int* g_exp,
                        const int* g_off, int x_div, int* err, cudaStream_t stream);
int vg_gemm_tc_grouped(const void* wt, const float* row_scale, const void* x_f16, int x_rows, int ldx, void* out, int out_f32,
                       int M, int K, int ldo, int wfmt, int bn, int max_items, const int* g_exp, const int* g_off,
                       const int* g_cnt, const int* tilemap, const int* n_items, int x_div, int* err, cudaStream_t stream);
int vg_gemm_tc_resident_ctas(int wfmt);
int vg_gemm_tc_set_debug(int dbg, long long* trace_buf);   // profiling builds only (-DVG_TRACE), else -1
int vg_gemm_simt(const void* wq, const void* scales, const float* row_scale, const void* x_f16, void* out, int out_f32,
                 int M, int K, int N, int ldx, int ldo, int wfmt, cudaStream_t stream);

int vg_add_rmsnorm(void* res, const void* delta, const float* w, void* out_f16, void* out_bf16, int N, int h, float eps,
                   int plus_one, int ld_res, int ld_delta, cudaStream_t stream);
int vg_attn_prep(const void* qkv, int ld_qkv, const float* q_norm, const float* k_norm, const int* pos, const int* slot,
                 const int* kv_row, void* q_out, void* kc, void* vc, int N, int nh, int nkv, int hd, int rdim,
                 int max_seq, float eps, float theta, int gated, void* k_scale, void* v_scale, cudaStream_t stream);
int vg_swiglu(const void* gu, void* out_f16, int N, int I, int ld, cudaStream_t stream);
int vg_cast_f16(const void* in, int in_is_f32, void* out_f16, long long total, cudaStream_t stream);
int vg_embed_gather(const void* table, const void* scales, const float* row_scale, const int* tok, void* out, int N,
                    int h, int wfmt, cudaStream_t stream);

int vg_attn_decode(const void* q, const void* kc, const void* vc, const int* lens, const int* slots, const int* base,
                   const int* path, int path_ld, float* part, int N, int nh, int nkv, int hd, int max_seq, int ns_grid,
                   int direct, const void* gate, int ld_gate, void* out, cudaStream_t stream);
// Tensor-core form of vg_attn_decode for head_dim 256, bf16 cache, no row indirection: one pass over the keys per KV
// head (all of its query heads, at most 16, share the fetched tiles). `block_table` (optional) makes the cache a pool
// of 128-key pages.
int vg_attn_decode_tc(const void* q, const void* kc, const void* vc, long long cache_rows, const int* lens, const int* slots,
                      const int* block_table, int bt_ld, float* part, int N, int nh, int nkv, int hd, int max_seq, int ns_grid,
                      const void* gate, int ld_gate, void* out, int* err, cudaStream_t stream);
int vg_attn_transpose_v(const void* vc, void* vT, int slot, int nkv, int hd, int max_seq, int len, int vt_cap,
                        cudaStream_t stream);
int vg_attn_prefill_tc(const void* q, int q_cap, const void* kc, const void* vT, int vt_cap, int slot, int nkv, int nh,
                       int hd, int max_seq, int pos0, int n, float scale, const void* gate, int ld_gate, void* out_f16,
                       int* err, cudaStream_t stream);
int vg_attn_decode_q4(const void* q, const void* kq, const void* vq, const void* ks, const void* vs, const int* lens,
                      const int* slots, const int* base, const int* path, int path_ld, float* part, int N, int nh, int nkv,
                      int hd, int max_seq, int ns_grid, int direct, const void* gate, int ld_gate, void* out,
                      cudaStream_t stream);
int vg_kv_q4_dequant(const void* codes, const void* scales, int slot, int nkv, int hd, int max_seq, int len, void* out_rows,
                     void* out_transposed, int t_cap, cudaStream_t stream);
long long vg_attn_scratch_floats(int N, int nh, int hd, int ns_grid);

int vg_gdn_conv(const void* x, int ldx, float* state, const float* w, const int* in_slot, const int* parent,
                const int* out_slot, float* out, int N, int conv_dim, int ck, int phase, cudaStream_t stream);
int vg_gdn_conv_chain(const void* x, int ldx, float* state, const float* w, const int* in_slot, const int* parent,
                      const int* out_slot, float* out, int N, int conv_dim, int ck, cudaStream_t stream);
int vg_gdn_prefill(const float* qkv, const void* proj, int ldp, int off_z, int off_b, int off_a, float* S,
                   const float* A_log, const float* dt_bias, const float* norm_w, int t0, int tn, const int* in_slot,
                   const int* out_slot, void* out_f16, int nk, int nv, int kd, int vd, float eps, float* o_scratch,
                   int split, cudaStream_t stream);
// Chunked (tensor-core) form of vg_gdn_prefill: 64-token chunks, tf32 MMAs, fp32 state. `work` is 1024-byte aligned
// scratch of vg_gdn_chunk_work_bytes(tn, nv) bytes, `o_raw` fp32 scratch of (t0 + tn) * nv * vd elements. The state is
// read from slot in_slot[t0] and written to out_slot[t0 + tn - 1] when that is >= 0 (no other checkpoints).
long long vg_gdn_chunk_work_bytes(int tn, int nv);
int vg_gdn_chunk_prefill(const float* qkv, const void* proj, int ldp, int off_z, int off_b, int off_a, float* S,
                         const float* A_log, const float* dt_bias, const float* norm_w, int t0, int tn, const int* in_slot,
                         const int* out_slot, void* out_f16, int nk, int nv, int kd, int vd, float eps, void* work,
                         float* o_raw, int* err, cudaStream_t stream);
int vg_gdn_step(const float* qkv, const void* proj, int ldp, int off_z, int off_b, int off_a, float* S, const float* A_log,
                const float* dt_bias, const float* norm_w, const int* chain_start, const int* chain_len, int n_chains,
                const int* in_slot, const int* parent, const int* out_slot, void* out_f16, int nk, int nv, int kd, int vd,
                float eps, void* bq, int ldb, void* sfb, float* g0, unsigned int* col_ctr, int* err, cudaStream_t stream);

int vg_argmax(const float* logits, int N, int V, int ld, int* out, float* out_val, int idx_offset, cudaStream_t stream);
int vg_penalty(float* logits, int N, int V, int ld, const int* toks, const int* counts, const int* n_toks, int max_toks,
               const float* rep, const float* pres, const float* freq, int idx_offset, cudaStream_t stream);
int vg_topk_chunks(int V);
int vg_topk_local(const float* logits, int N, int V, int ld, const float* temp, const int* top_k, int idx_offset,
                  void* cand_chunks, void* out_cand, cudaStream_t stream);
int vg_nucleus_finish(const void* lists, int n_lists, int row_stride_pairs, int N, const float* temp, const int* top_k,
                      const float* top_p, const float* u, int* out_tok, int* ids, float* probs, int* n_keep,
                      cudaStream_t stream);
int vg_spec_verify(const int* ids, const float* probs, const int* n_keep, const int* drafts, const float* u_acc,
                   const float* u_ver, const int* col0, const int* nd, int n_lanes, int* result, cudaStream_t stream);
int vg_nucleus(const float* logits, int N, int V, int ld, const float* temp, const int* top_k, const float* top_p,
               const unsigned* seed, int* out_tok, int* ids, float* probs, int* n_keep, cudaStream_t stream);
int vg_nll(const float* logits, int N, int V, int ld, const int* target, float* out, cudaStream_t stream);

int vg_moe_router(const float* logits, int N, int E, int K, int sigmoid_mode, const float* bias, int norm, float scaling,
                  int e_base, int n_local, int* ids, float* wts, int* g_exp, int* g_off, int* g_cnt, cudaStream_t stream);
int vg_moe_sort(const int* ids, int P, int e_base, int n_local, int bn, int* cnt, int* cursor, int* g_exp, int* g_off,
                int* g_cnt, int* tilemap, int* n_items, int* perm, int* inv, int* total, cudaStream_t stream);
int vg_moe_gather(const void* x_f16, int ldx, const int* perm, const int* total, int max_rows, int topk, int h,
                  void* out_f16, cudaStream_t stream);
int vg_moe_combine(const void* y, int ldy, const int* inv, const float* wts, int N, int topk, const void* shared,
                   const float* gate_logit, void* out, int h, cudaStream_t stream);
int vg_moe_combine_push(const void* y, int ldy, const int* inv, const float* wts, int N, int topk, const void* shared,
                        const float* gate_logit, int h, const VgCommCtx* ctx, cudaStream_t stream);
int vg_moe_add_shared(void* out, const void* shared, const float* gate_logit, int N, int h, cudaStream_t stream);

int vg_comm_alloc(void** ptr, unsigned long long bytes);
int vg_comm_free(void* ptr);
int vg_comm_export(void* ptr, void* handle64);
int vg_comm_import(const void* handle64, void** ptr);
int vg_comm_close(void* ptr);
int vg_comm_handle_bytes(void);
int vg_comm_allreduce(const VgCommCtx* ctx, const void* in, int in_is_f32, void* out_bf16, float* out_f32, long long n,
                      cudaStream_t stream);
int vg_comm_allreduce_multimem(const VgCommCtx* ctx, void* mc_buf, long long n, cudaStream_t stream);
int vg_comm_allgather_small(const VgCommCtx* ctx, const void* in, void* out, int bytes, cudaStream_t stream);
int vg_comm_argmax_merge(const VgCommCtx* ctx, const float* val, const int* idx, int ncols, float* scratch_pairs,
                         float* gathered, int* out, cudaStream_t stream);
int vg_comm_wait_timeout_probe(const VgCommCtx* ctx, unsigned long long budget_ns, cudaStream_t stream);

const char* vg_build_id(void);

#ifdef __cplusplus
}
#endif

// C ABI of libadana_b200.so.  Every entry point takes raw device pointers and the CUDA
// stream (as void*) to launch on, returns 0 on success (a negative value for a rejected
// argument, a positive cudaError_t for a failed launch) and never allocates device memory
// unless its comment says so.  Python binds these with ctypes (adana_b200/ops/_lib.py).
#pragma once
#include <stdint.h>

// GEMM epilogues
enum {
  EPI_BF16 = 0,       // C(bf16) = alpha * acc
  EPI_GELU_DUAL = 1,  // C(bf16) = acc (pre-activation), C2(bf16) = gelu(acc)
  EPI_RESID_F32 = 2,  // C(f32)  = R(f32) + alpha * acc
  EPI_DGELU = 3,      // C(bf16) = acc * gelu'(R(bf16))
  EPI_F32 = 4,        // C(f32)  = beta * C + alpha * acc
  EPI_SWIGLU = 5,     // B = [gate; up] rows; C(bf16)=[gate|up] pre-activations, C2 = silu(g)*u
  EPI_DSWIGLU = 6,    // acc = dH; R = [gate|up]; C = [dGate|dUp]
  EPI_AXPBY_BF16 = 7, // C(bf16) = alpha * acc + beta * R(bf16); C may alias R
  EPI_F32_ATOMIC = 8, // C(f32) += alpha * acc with vector atomics (internal: stream-K partial tiles)
  EPI_F32_RS = 9,     // rows added into the fp32 buffer of the rank that owns them (adana_gemm_bf16_reduce_scatter)
  EPI_BF16_PUSH = 10, // rows stored (bf16) into this rank's slot at the rank that owns them (same entry point)
};

#ifdef __cplusplus
extern "C" {
#endif

// D = epilogue(A * B^T), bf16 operands, fp32 accumulate on tcgen05 tensor cores.
// a_mn / b_mn select MN-major operands (see gemm_tcgen05.cu).  ld* are row pitches in elements.
// GEMM fused with the reduce-scatter that follows a row-parallel linear: this rank holds a K-slice of the operands,
// A [M, K] and B [N, K] (both K-major); rank r keeps output rows [r * rows_per_rank, (r + 1) * rows_per_rank).
// Row tiles are taken starting at the rows of rank my_rank + 1, so the ranks do not all send to one destination.
//  push_bf16 = 1 (preferred): the epilogue STORES this rank's partial rows (bf16, plain 16-byte stores, over NVLink
//   for remote rows) into slot my_rank of the owner's slot array C_ranks[owner] ([n_ranks, rows_per_rank, ldc] bf16).
//   After a barrier over the ranks the owner sums its n_ranks slots in fp32 in a fixed order (adana_sum_slots_bf16):
//   deterministic, nothing to zero, no atomics.  The caller synchronises the ranks before the launch too, so that no
//   slot is overwritten while its owner still reads it.
//  push_bf16 = 0: the partial product is ADDED (`red.global.add.v4.f32`) into C_ranks[owner] ([rows_per_rank, ldc]
//   fp32, zero-filled or pre-loaded by its owner before a barrier); bound by the L2's fp32 atomic rate (~0.5 TB/s).
int adana_gemm_bf16_reduce_scatter(const void* A, const void* B, void* const* C_ranks, int n_ranks, int my_rank,
                                   int rows_per_rank, int M, int N, int K, long long lda, long long ldb,
                                   long long ldc, float alpha, int push_bf16, int* status, void* stream);
// out [rows, N] (fp32, pitch ld_out) = (resid ? resid : 0) + sum over s < n_slots of slots[s][rows][N] (bf16, pitch
// ld_slot), summed in fp32 in slot order; out_bf16 (optional) receives a bf16 copy.  N a multiple of 8.
int adana_sum_slots_bf16(const void* slots, int n_slots, int rows, int N, long long ld_slot, float* out,
                         long long ld_out, const float* resid, long long ld_resid, void* out_bf16,
                         long long ld_out16, void* stream);
// Pull-style reduce-scatter of bf16 partial matrices: rank r's partial product P_r [M, N] (pitch ld) sits at
// partial_ptrs[r] (local or peer memory); out = (resid or 0) + sum over r of P_r[first_row : first_row + rows], fp32
// accumulation in rank order, the peers' rows read over NVLink.  Call between two barriers over the ranks.
int adana_p2p_reduce_scatter_bf16(const unsigned long long* partial_ptrs, int n_ranks, long long first_row, int rows,
                                  int N, long long ld, float* out, long long ld_out, const float* resid,
                                  long long ld_resid, void* out_bf16, long long ld_out16, void* stream);
// Variable-size all-to-all of rows over peer memory, pull style (expert-parallel dispatch / combine): every rank has
// published a row buffer sorted by destination (buf_ptrs[p]) and an int32 table (tab_ptrs[p]) of 2 * world +
// world * segs_per_rank entries: first row and row count of the group held for each rank, then the row counts of the
// segments inside the groups, destination rank major; rank `me` copies the rows every peer holds for it, peers in rank order, into
// `out` (nullptr: counts only) and the peers' counts for it into out_counts [world * segs_per_rank].  More than
// max_rows_out rows: the copy is clamped and *status set.  Call between two barriers over the ranks.
int adana_p2p_all_to_all_pull(const unsigned long long* buf_ptrs, const unsigned long long* tab_ptrs, int me,
                              int world, int segs_per_rank, long long row_bytes, void* out, long long max_rows_out,
                              int* out_counts, int* status, void* stream);

// All-gather fused into the GEMM.  The weight W is split by rows over `n_shards` ranks: rank r holds rows
// [row_starts[r], row_starts[r+1]) (multiples of 32; nullptr = equal slices of rows_per_shard rows) at B_shards[r]
// (local or peer memory, row pitch ldb).  b_mn = 0: C[M,N] = epi(A[M,K] * W[N,K]^T); b_mn = 1: C[M,N] = epi(A[M,K] *
// W[K,N]).  Each CTA pair fetches its B tiles straight from the owning rank — whole-tile TMA boxes inside a slice,
// 32-row boxes where a tile straddles two slices — so no gathered copy of W exists.  epi: EPI_BF16, EPI_GELU_DUAL,
// EPI_RESID_F32 (b_mn = 0) or EPI_BF16, EPI_DGELU (b_mn = 1).
// With `stage` (a [rows of W, ldb] bf16 matrix of this rank), `flags` (64 + rows / 8 ints) and `my_rank`, extra
// warps of the same kernel copy the remote slices into `stage` once, while the tiles on my_rank's own slice run,
// and the other tiles read the staged copy: every weight byte crosses the link once.  Slices must then be cut on
// multiples of 128 rows (64 for b_mn = 1), and launches that share `stage`/`flags` be ordered on one stream.
int adana_gemm_bf16_gather(const void* A, const void* const* B_shards, int n_shards, int rows_per_shard,
                           const int* row_starts, void* C, int M, int N, int K, long long lda, long long ldb,
                           long long ldc, int b_mn, int epi, void* C2, long long ldc2, const void* R, long long ldr,
                           float alpha, int my_rank, void* stage, int* flags, int* status, void* stream);
// Tile shape policy of adana_gemm_bf16: 0 = per shape (default), 1 = one CTA per 128x256 tile,
// 2 = CTA pair (cta_group::2) per 256x256 tile, with stream-K for fp32 outputs whose whole-tile
// waves would idle the machine, 3 = CTA pair without stream-K.  Returns the previous mode.
int adana_gemm_set_mode(int mode);
int adana_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                    long long ldb, long long ldc, int a_mn, int b_mn, int epi, void* C2,
                    long long ldc2, const void* R, long long ldr, float alpha, float beta,
                    int b_off2, int* status, void* stream);

// ---- normalisation (norm.cu) -------------------------------------------------------------
// y(bf16|f32) = norm(x(f32|bf16)) * w ; kind 0 = LayerNorm (mean-subtracting, weight only),
// kind 1 = RMSNorm.  Saves mean/rstd (fp32, one per row) for backward.
int adana_norm_fwd(const void* x, int x_is_bf16, const float* w, void* y, int y_is_bf16,
                   float* mean, float* rstd, int rows, int cols, float eps, int kind,
                   void* stream);
// dx(f32) (+)= d norm / dx ; dw_partial[blocks, cols] fp32 partial sums reduced by
// adana_colsum_f32.  accumulate_dx: dx += result (residual-stream gradient accumulation).
int adana_norm_bwd(const void* dy, int dy_is_bf16, const void* x, int x_is_bf16, const float* w,
                   const float* mean, const float* rstd, float* dx, int accumulate_dx,
                   float* dw_partial, int n_partial_rows, int rows, int cols, int kind,
                   void* dx_bf16 /*optional bf16 copy of the final dx*/, void* stream);
int adana_colsum_f32(const float* partial, int n_partial_rows, int cols, float* out,
                     int accumulate, void* stream);

// ---- per-head QK-norm + rotary embedding (rope.cu) --------------------------------------------
// q/k are read in place from the fused projection output: element (token, head h, i) of q is at
// qkv[token * row_stride + q_off + h * q_hstride + i].  kind: 0 LayerNorm, 1 RMSNorm, 2 none.
int adana_qknorm_rope_fwd(const void* qkv, long long row_stride, int q_off, int q_hstride,
                          int k_off, int k_hstride, const float* wq, const float* wk,
                          const float* freqs, void* q_out, void* k_out, long long n_tokens, int S,
                          int Hq, int Hk, int hd, float eps, int kind, void* stream);
int adana_qknorm_rope_bwd(const void* dq, const void* dk, const void* qkv, long long row_stride,
                          int q_off, int q_hstride, int k_off, int k_hstride, const float* wq,
                          const float* wk, const float* freqs, void* dqkv, float* dwq_partial,
                          float* dwk_partial, int n_partial, long long n_tokens, int S, int Hq,
                          int Hk, int hd, float eps, int kind, int dq_is_f32, void* stream);
int adana_sigmoid_gate_fwd(const void* a, const void* gate, long long gate_row_stride, int gate_off,
                           int gate_hstride, void* out, long long n_tokens, int H, int hd,
                           void* stream);
int adana_sigmoid_gate_bwd(const void* dout, const void* a, const void* gate,
                           long long gate_row_stride, int gate_off, int gate_hstride, void* da,
                           void* dgate_base, long long n_tokens, int H, int hd, void* stream);

// ---- embedding (embedding.cu) ----------------------------------------------------------------
int adana_embedding_fwd(const long long* idx, const void* table, int table_is_bf16, float* out,
                        int n_tokens, int dim, int vocab, void* stream);
int adana_embedding_bwd(const long long* idx, const float* dout, float* dtable, int n_tokens,
                        int dim, int vocab, void* stream);

// ---- cross entropy over a chunk of fp32 logits (ce.cu) -----------------------------------------
int adana_ce_fwd_bwd(float* logits, long long ld, const long long* targets, int rows, int vocab,
                     float z_coeff, float grad_scale, void* dlogits_bf16, long long ldd,
                     float* sums /*[4]: ce, lse^2, correct, valid*/, float* lse_out,
                     void* stream);
// The same over bf16 logits; dlogits_bf16 may be the logits buffer itself (in place) or null.
int adana_ce_fwd_bwd_bf16(void* logits, long long ld, const long long* targets, int rows, int vocab, float z_coeff,
                          float grad_scale, void* dlogits_bf16, long long ldd, float* sums, float* lse_out,
                          void* stream);

// ---- optimizer (optim.cu) ----------------------------------------------------------------------
struct AdanaOptHyper {
  float lr;            // scheduled learning rate of the group (g2 = g3 = lr)
  float alpha;         // delta / (delta + t)
  float step;          // t (1-based)
  float one_minus_kappa;
  float clipsnr;       // < 0: no clipping
  float eps;
  float gamma3;        // gamma_3_factor
  float wd_factor;     // 1 - wd * sched / (1 + t / wd_ts)   (already folded on the host)
  float grad_scale;    // multiplies the raw gradient (1/acc_steps, 1/world); the clip
                       // coefficient is read from clip_coef_ptr on the device
  int kind;            // 0 adana/dana-mk4, 1 dana-star(-mk4), 2 adamw, 3 adamw + independent decay,
                       // 4 ademamix (coupled decay), 5 ademamix + independent decay
  float beta1, beta2, bc1, bc2;  // adamw and ademamix
  float beta3;         // ademamix: decay of the slow EMA at this step (after its warm-up); `alpha` is the mixing
                       // coefficient at this step; the slow EMA lives in the `tau` buffer
  float wd_coupled;    // ademamix kind 4: weight decay added to the update (p -= lr * (update + wd * p))
};
int adana_opt_step(float* p, const float* g, float* m, float* v, float* tau, void* p_bf16,
                   long long n, const struct AdanaOptHyper* h, const float* clip_coef_ptr,
                   float* diag /*[4] or null*/, void* stream);
int adana_sumsq_f32(const float* x, long long n, float* out /*accumulates*/, void* stream);
int adana_clip_coef(const float* sumsq, float norm_scale, float max_norm, float* out /*[2]: coef, norm*/,
                    void* stream);

// ---- peer-memory collectives (comm_p2p.cu); *_ptrs are arrays of `world` device addresses, one per rank ----
int adana_p2p_barrier(const unsigned long long* flag_ptrs, int rank, int world, int slot_base, unsigned int seq,
                      unsigned long long timeout_ns, int* status, void* stream);
int adana_p2p_reduce_scatter(const unsigned long long* grad_ptrs, int world, long long shard_off, long long n,
                             float* out, float* sumsq, void* stream);
// Per-unit "ready" flags and the collectives that wait for them (see comm_p2p.cu).
int adana_p2p_signal(const unsigned long long* flag_ptrs, int rank, int world, int slot, unsigned int seq,
                     void* stream);
int adana_p2p_reduce_scatter_flag(const unsigned long long* src_ptrs, int wire_bf16, const void* my_flags,
                                  unsigned int seq, int world, long long shard_off, long long n, float* out,
                                  float* sumsq, unsigned long long timeout_ns, int* status, void* stream);
int adana_p2p_all_reduce_flag(const unsigned long long* src_ptrs, int wire_bf16, const unsigned long long* dst_ptrs,
                              const void* my_flags, unsigned int seq, int world, long long slice_off, long long n,
                              float* sumsq, unsigned long long timeout_ns, int* status, void* stream);
int adana_p2p_publish_f32(const unsigned long long* slot_ptrs, int rank, int world, const float* value, void* stream);
int adana_p2p_push_f32(const float* src, const unsigned long long* dst_ptrs, int world, long long dst_off, long long n,
                       void* stream);
int adana_clip_coef_multi(const float* partials, int world, float norm_scale, float max_norm, float* out, void* stream);
int adana_p2p_opt_step_push(float* p, const float* g, float* m, float* v, float* tau,
                            const unsigned long long* weight_ptrs, int world, long long push_off, long long n,
                            const struct AdanaOptHyper* h, const float* clip_coef_ptr, void* stream);

// ---- attention (attention_tcgen05.cu) ----
int adana_attn_fwd(const void* q, const void* k, const void* vbase, long long ldv, int v_hstride, void* out,
                   float* lse2, int B, int S, int Hq, int Hk, int hd, float scale, int* status, void* stream);
int adana_attn_bwd(const void* dout, const void* q, const void* k, long long ldv, int v_hstride, const void* vbase,
                   const void* out, const float* lse2, float* delta, float* dq_acc, void* dk, long long lddv,
                   int dv_hstride, void* dvbase, int B, int S, int Hq, int Hk, int hd, float scale, int* status,
                   void* stream);

// ---- utility -------------------------------------------------------------------------------------
int adana_cast_f32_to_bf16(const float* src, void* dst, long long n, void* stream);
// ---- distributed Muon chain (muon_chain.cu) ----------------------------------------------------------------------
// Segment tables are device arrays of 32-byte entries {int64 a, b; int32 kind, group; float shape_factor; int32 mat}.
int adana_muon_parts(void);
int adana_muon_momentum(const float* g, float* buf, void* ns_out, const void* segs, int n_segs, const float* clip,
                        float gscale, float mu, int nesterov, float* parts, void* stream);
int adana_muon_pull(const unsigned long long* staged_ptrs, const unsigned long long* parts_ptrs, int world,
                    long long shard_len, long long off, long long n, int mat, float eps, void* X, const void* flags,
                    unsigned int seq, unsigned long long timeout_ns, int* status, void* stream);
int adana_muon_push(const void* X, const unsigned long long* upd_ptrs, int world, long long shard_len, long long off,
                    long long n, void* stream);
int adana_muon_apply(float* p, const float* g, const void* upd, float* m1, float* m2, const void* segs, int n_segs,
                     const float* hyper, const float* clip, const unsigned long long* weight_ptrs, int n_dst,
                     long long push_off, long long max_seg_len, const void* flags, unsigned int seq, int world,
                     unsigned long long timeout_ns, int* status, void* stream);
int adana_version(void);

// ---- attention JVP (attention_jvp_tcgen05.cu) ---------------------------------------------------
// Primal output and forward-mode tangent of causal attention in one pass.  q, tq [T, Hq, hd];
// k, tk, v, tv [T, Hk, hd]; out, tout [T, Hq*hd]; contiguous bf16, T = B*S, S % 128 == 0, hd 64 | 128.
int adana_attn_jvp(const void* q, const void* tq, const void* k, const void* tk, const void* v,
                   const void* tv, void* out, void* tout, int B, int S, int Hq, int Hk, int hd,
                   float scale, int* status, void* stream);

#ifdef __cplusplus
}
#endif

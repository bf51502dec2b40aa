// C entry points of the sm_100a kernel library. Every function enqueues work on `stream` and returns 0 on a
// successful launch, a negative code for a rejected argument or a failed launch. Device-side failures
// (bounded waits that expired, capacity overflow) are reported through the `status` word, see common.cuh.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---- GEMM family (gemm.cu) ----
int llmt_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                   int a_mn, int b_mn, int out_f32, int accumulate, int* status, int max_ctas, cudaStream_t stream);
int llmt_gemm_bf16_fused(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                         int a_mn, int b_mn, int out_f32, int accumulate, int job_kind, int job_nsrc,
                         const void* const* job_src, void* job_dst, long long job_n, int job_accumulate,
                         const uint32_t* wait_flags, int n_wait, uint32_t wait_value, int* status, cudaStream_t stream);
int llmt_gemm_bf16_tp(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                      int b_mn, int accumulate, int mode, int world, int rank, uint32_t epoch, const void* const* peer_src,
                      const uint32_t* flags, uint32_t* const* peer_flags, uint32_t* counters, float* acc, void* out,
                      const void* residual, int* status, cudaStream_t stream);
int llmt_grouped_gemm_bf16(const void* A, const void* B, void* C, const int* seg_offsets, int num_groups, int M_padded,
                           int N, int K, int64_t lda, int64_t ldc, int b_mn, int out_f32, int* status,
                           cudaStream_t stream);
int llmt_grouped_wgrad_bf16(const void* A, const void* B, void* C, const int* seg_offsets, int num_groups,
                            int rows_padded, int M, int N, int64_t lda, int64_t ldb, int out_f32, int accumulate,
                            int* status, cudaStream_t stream);

// ---- memory-bound kernels (elementwise.cu) ----
int llmt_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* sum_out, float* rstd, int T, int D,
                     float eps, cudaStream_t st);
int llmt_rmsnorm_bwd_partials(int T);
int llmt_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx,
                     float* dw_partial, float* dw_f32, void* dw_bf16, int accumulate, int T, int D, cudaStream_t st);
int llmt_qk_norm_rope_fwd(const void* x, int64_t tok_stride, const void* w, const float* cosb, const float* sinb, void* y,
                          int64_t y_tok_stride, float* rstd, int T, int H, int HD, float eps, cudaStream_t st);
int llmt_qk_norm_rope_bwd_partials(int T, int H);
int llmt_qk_norm_rope_bwd(const void* dy, int64_t dy_tok_stride, const void* x, int64_t tok_stride, const void* w,
                          const float* cosb, const float* sinb, const float* rstd, void* dx, int64_t dx_tok_stride,
                          float* dw_partial, float* dw_f32, void* dw_bf16, int accumulate, int T, int H, int HD,
                          cudaStream_t st);
int llmt_attn_rows_probs(const float* s, const float* lse, void* p, int64_t rows, int C, int n, int diag, float scale,
                         int causal, cudaStream_t st);
int llmt_attn_rows_ds(const float* dp, const void* p, const float* delta, void* ds, int64_t rows, int C, cudaStream_t st);
int llmt_swiglu_fwd(const void* gate, const void* up, void* out, int64_t T, int F, int64_t ld_in, int64_t ld_out,
                    const int* row_limit, cudaStream_t st);
int llmt_swiglu_bwd(const void* dout, const void* gate, const void* up, void* dgate, void* dup, int64_t T, int F,
                    int64_t ld_in, int64_t ld_dout, int64_t ld_dg, const int* row_limit, cudaStream_t st);
int llmt_ce_fwd_bwd(void* logits, const int64_t* labels, float* row_loss, float* row_lse, int rows, int V, int64_t ld,
                    const float* grad_scale_ptr, float grad_scale, int ignore_index, int write_grad, cudaStream_t st);
int llmt_adamw(float* p32, void* p16, const void* g, int g_is_bf16, float* m, float* v, int64_t n, float lr, float b1,
               float b2, float eps, float wd, int step, const float* clip_coef, float grad_scale, int decoupled,
               cudaStream_t st);
int llmt_sqnorm_scratch_floats();
int llmt_sqnorm(const void* x, int is_bf16, int64_t n, float* scratch, float* out, int accumulate, cudaStream_t st);
int llmt_clip_coef(const float* total_sq, float max_norm, float* clip_coef, float* norm_out, int* finite, cudaStream_t st);

// ---- expert-parallel token exchange over peer memory (ep_comm.cu) ----
int llmt_ep_exchange(const int64_t* flat, int64_t ncopies, int E, int R, int me, void* const* tables, void* const* flags,
                     uint32_t epoch, int cap, int* seg_offsets, int* totals, int* send_off, int* status, cudaStream_t st);
int llmt_ep_plan(const int64_t* flat, int64_t ncopies, int E, int R, const int* send_off, int* drank, int* drow, cudaStream_t st);
int llmt_ep_push_rows(const void* src, const float* scale, const int* drank, const int* drow, void* const* bufs, int R, int cap,
                      int64_t ncopies, int k, int D, const void* other, float* dot_out, int* status, cudaStream_t st);
int llmt_ep_pull_rows(void* const* bufs, int R, const int* drank, const int* drow, const float* w, void* out, void* keep, int cap,
                      int T, int k, int D, cudaStream_t st);
int llmt_ep_clone_rows(const void* src, void* dst, const int* seg_offsets, const int* totals, int G, int D, int zero_pad,
                       cudaStream_t st);

// ---- MoE routing and token movement (moe.cu) ----
int llmt_router_topk(const float* logits, const float* bias, float* weights, int64_t* indices, float* counts, float* denom,
                     int T, int E, int k, int score_fn, int renorm, float route_scale, cudaStream_t st);
int llmt_router_topk_bwd(const float* logits, const float* dweights, const int64_t* indices, const float* denom, float* dlogits,
                         int T, int E, int k, int score_fn, int renorm, float route_scale, cudaStream_t st);
int llmt_permute_rows(const void* x, const int64_t* dest, void* rows, int64_t ncopies, int k, int D, cudaStream_t st);
int llmt_combine_rows(const void* y, const int64_t* dest, const float* w, void* out, int T, int k, int D, cudaStream_t st);
int llmt_combine_bwd(const void* dout, const void* y, const int64_t* dest, const float* w, void* dy, float* dw, int64_t ncopies,
                     int k, int D, cudaStream_t st);

// ---- peer-memory communication (comm.cu) ----
int llmt_side_job(int kind, int nsrc, const void* const* src, void* dst, long long n, int accumulate,
                  const uint32_t* wait_flags, int n_wait, uint32_t wait_value, int ctas, int* status, cudaStream_t st);
int llmt_signal_peers(uint32_t* const* peer_flags, int npeers, int slot, uint32_t value, cudaStream_t st);
int llmt_wait_flags(const uint32_t* flags, int n, uint32_t value, int site, uint32_t max_polls, int* status,
                    cudaStream_t st);

// ---- vocabulary-parallel loss and embedding over peer memory (vocab_parallel.cu) ----
int llmt_ce_vocab_parallel(void* logits, const int64_t* labels, float* row_loss, int rows, int Vr, int64_t ld,
                           int64_t vocab_start, int R, int me, void* const* stats, void* const* flags, int cap, uint32_t epoch,
                           float grad_scale, int ignore_index, int write_grad, int* status, cudaStream_t st);
int llmt_vp_embed_scatter(const int64_t* ids, const void* w, int64_t vstart, int64_t vend, void* const* out, int R, int T,
                          int chunk, int D, cudaStream_t st);

// ---- attention (attention.cu) ----
// q [Tq, Hq, HD], k/v [Tk, Hkv, HD] bf16 with token strides in elements; varlen via cu_seqlens (device int32).
// tiles: device int32 [num_tiles][4] = {q_row_begin, q_row_end, k_row_begin, k_causal_end_for_first_row}; see attention.cu.
int llmt_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int* tiles, int num_tiles,
                  int Tq, int Tk, int Hq, int Hkv, int HD, int64_t q_stride, int64_t k_stride, int64_t v_stride,
                  int64_t o_stride, float scale, int causal, int* status, cudaStream_t st);
// Same contract; one CTA per (q tile, pair of query heads of one key/value group). Needs an even group size.
int llmt_attn_fwd_pair(const void* q, const void* k, const void* v, void* o, float* lse, const int* tiles, int num_tiles,
                       int Tq, int Tk, int Hq, int Hkv, int HD, int64_t q_stride, int64_t k_stride, int64_t v_stride,
                       int64_t o_stride, float scale, int causal, int* status, cudaStream_t st);
int llmt_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                  float* delta, void* dq, void* dk, void* dv, const int* q_tiles, int num_q_tiles, const int* k_tiles,
                  int num_k_tiles, int Tq, int Tk, int Hq, int Hkv, int HD, int64_t q_stride, int64_t k_stride,
                  int64_t v_stride, int64_t o_stride, int64_t do_stride, int64_t dq_stride, int64_t dk_stride,
                  int64_t dv_stride, float scale, int causal, int pass, int* status, cudaStream_t st);
// Single-kernel backward (attention_bwd.cu): dK, dV and dQ from one walk per key tile; dQ is summed in the fp32
// accumulator dq_acc [Tq, Hq, HD] (cleared when `first`, cast into dq when `last`).
int llmt_attn_bwd_fused(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                        float* delta, float* dq_acc, void* dq, void* dk, void* dv, const int* k_tiles, int num_k_tiles,
                        int Tq, int Tk, int Hq, int Hkv, int HD, int64_t q_stride, int64_t k_stride, int64_t v_stride,
                        int64_t o_stride, int64_t do_stride, int64_t dq_stride, int64_t dk_stride, int64_t dv_stride,
                        float scale, int causal, int first, int last, int* status, cudaStream_t st);

#ifdef __cplusplus
}
#endif

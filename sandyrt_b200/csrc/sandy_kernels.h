// C declarations of every kernel launcher of this folder.  Each `<name>.cu` builds into one
// shared library that exports the functions listed under its name; all take raw device pointers
// and a stream, launch on that stream (so a launch can be captured in a CUDA graph) and return 0,
// SANDY_ERR_UNSUPPORTED (-1: sizes or dtypes the kernel refuses), SANDY_ERR_ARGUMENT (-2) or a
// cudaError_t.  dtype codes: 0 = float32, 1 = bfloat16.  `status` arguments are device ints in
// which kernels raise bits instead of faulting (bad token ids, pages that do not exist, waits
// that ran out).
#pragma once

#include <cuda_runtime.h>

#include "matrix_state.h"

#ifdef __cplusplus
extern "C" {
#endif

/* embed.cu */
int sandy_embed_pos(const int* ids, const int* pos, const void* wte, const void* wpe, void* out, int n_tokens, int width,
                    int vocab, int n_pos, int table_dtype, int out_dtype, int* status, cudaStream_t stream);
int sandy_device_sm_count(void);
int sandy_spin(long long nanoseconds, cudaStream_t stream);

/* norm.cu */
int sandy_layernorm(const void* x, const void* gamma, const void* beta, void* out, const int* rows, int n_rows, int width,
                    float eps, int in_dtype, int w_dtype, int out_dtype, cudaStream_t stream);

/* gemm_simt.cu */
int sandy_gemm_simt(const void* a, const void* w, const void* bias, const float* residual, void* out, int M, int N, int K,
                    int lda, int ldw, int ldr, int ldc, int w_out_in, int act, int a_dtype, int w_dtype, int out_dtype,
                    cudaStream_t stream);

/* gemm_tc.cu, gemm_tc2.cu */
int sandy_gemm_tc(const void* a, const void* w, const void* bias, const float* residual, void* out, int M, int N, int K,
                  int lda, int ldw, int ldr, int ldc, int act, int out_dtype, int tile_n, void* k_cache, void* v_cache,
                  long long page_stride, const int* block_table, int max_blocks, const int* token_seq, const int* positions,
                  int q_cols, int kv_cols, int head_dim, int page_size, int num_pages, int* status, cudaStream_t stream);
int sandy_gemm_tc2(const void* a, const void* w, const void* bias, const float* residual, void* out, int M, int N, int K,
                   int lda, int ldw, int ldr, int ldc, int act, int out_dtype, int tile_n, void* k_cache, void* v_cache,
                   long long page_stride, const int* block_table, int max_blocks, const int* token_seq, const int* positions,
                   int q_cols, int kv_cols, int head_dim, int page_size, int num_pages, int* status, cudaStream_t stream);

/* gemm_skinny.cu */
int sandy_gemm_skinny_norm_limits(int* max_rows, int* max_k);
int sandy_gemm_skinny(const void* a, const float* x, int ldx, const void* gamma, const void* beta, float eps, const void* w,
                      const void* bias, const float* residual, void* out, int M, int N, int K, int lda, int ldw, int ldr,
                      int ldc, int act, int out_dtype, void* k_cache, void* v_cache, long long page_stride,
                      const int* block_table, int max_blocks, const int* token_seq, const int* positions, int q_cols,
                      int kv_cols, int head_dim, int page_size, int num_pages, int* status, cudaStream_t stream);

/* gemm_small.cu */
int sandy_gemm_small_splits(int N, int K);
int sandy_gemm_small(const void* a, const void* w, const void* bias, const float* residual, void* out, int M, int N, int K,
                     int lda, int ldw, int ldr, int ldc, int act, int out_dtype, void* k_cache, void* v_cache,
                     long long page_stride, const int* block_table, int max_blocks, const int* token_seq,
                     const int* positions, int q_cols, int kv_cols, int head_dim, int page_size, int num_pages, int* status,
                     cudaStream_t stream);

/* attention.cu */
int sandy_kv_append(const void* k_src, const void* v_src, int ld_src, void* k_cache, void* v_cache, long long page_stride,
                    const int* block_table, int max_blocks, const int* token_seq, const int* positions, int n_tokens,
                    int n_kv_heads, int head_dim, int page_size, int num_pages, int dtype, int* status, cudaStream_t stream);
int sandy_paged_attention(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
                          const int* block_table, int max_blocks, const int* token_seq, const int* positions, void* out,
                          int ld_out, int n_tokens, int n_heads, int n_kv_heads, int head_dim, int page_size, float scale,
                          int window, int num_pages, int dtype, int* status, cudaStream_t stream);

/* attention_decode.cu */
int sandy_decode_attention_cluster(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
                                   const int* block_table, int max_blocks, const int* token_seq, const int* positions,
                                   void* out, int ld_out, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                   int page_size, float scale, int window, int num_splits, int num_pages, int dtype,
                                   int* status, cudaStream_t stream);
long long sandy_decode_attention_scratch_floats(int n_tokens, int n_heads, int head_dim, int num_splits);
int sandy_decode_attention(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
                           const int* block_table, int max_blocks, const int* token_seq, const int* positions, void* out,
                           int ld_out, float* scratch, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                           int page_size, float scale, int window, int num_splits, int num_pages, int dtype, int* status,
                           cudaStream_t stream);

/* attention_decode_mma.cu */
int sandy_decode_attention_mma_max_keys(int num_splits, int page_size);
int sandy_decode_attention_mma(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
                               const int* block_table, int max_blocks, const int* token_seq, const int* positions, void* out,
                               int ld_out, int n_tokens, int n_heads, int n_kv_heads, int head_dim, int page_size, float scale,
                               int window, int num_splits, int num_pages, int max_keys, int* status, cudaStream_t stream);

/* attention_decode_bulk.cu */
int sandy_decode_attention_bulk(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
                                const int* block_table, int max_blocks, const int* token_seq, const int* positions,
                                void* out, int ld_out, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                int page_size, float scale, int window, int num_splits, int num_pages, int dtype,
                                int* status, cudaStream_t stream);

/* attention_prefill.cu, attention_prefill_tc.cu */
int sandy_prefill_attention(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
                            const int* block_table, int max_blocks, const int* q_start, const int* kv_before, void* out,
                            int ld_out, int n_seqs, int max_q_len, int n_heads, int n_kv_heads, int head_dim,
                            int page_size, float scale, int window, int num_pages, int* status, cudaStream_t stream);
int sandy_prefill_attention_tc(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
                               const int* block_table, int max_blocks, const int* q_start, const int* kv_before, void* out,
                               int ld_out, int n_seqs, int max_q_len, int n_heads, int n_kv_heads, int head_dim,
                               int page_size, float scale, int window, int num_pages, int* status, cudaStream_t stream);

/* the attention kernels with a sink per head (float32 [H]: exp(sink) joins the softmax's denominator) and a factor on
   each head's output (float32 [T, H]); either may be null.  The entry points above are these with both null. */
int sandy_paged_attention_ext(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
                              const int* block_table, int max_blocks, const int* token_seq, const int* positions, void* out,
                              int ld_out, int n_tokens, int n_heads, int n_kv_heads, int head_dim, int page_size, float scale,
                              int window, int num_pages, int dtype, const float* sink, const float* out_gate, int* status,
                              cudaStream_t stream);
/* ... and with two rules on the scores: softcap > 0 presses a score into softcap * tanh(score / softcap); chunk > 0
   lets a query see only the keys of its own chunk of positions (j >= pos - pos % chunk).  Zero switches a rule off. */
int sandy_paged_attention_cap(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
                              const int* block_table, int max_blocks, const int* token_seq, const int* positions, void* out,
                              int ld_out, int n_tokens, int n_heads, int n_kv_heads, int head_dim, int page_size, float scale,
                              int window, float softcap, int chunk, int num_pages, int dtype, const float* sink,
                              const float* out_gate, int* status, cudaStream_t stream);
/* ... and with a learned bias by distance: entry min(i - j, n_dist - 1) of the head's row of dist_bias (float32
   [H, n_dist]) joins the score of query i and key j after the scale and the cap.  Null: none. */
int sandy_paged_attention_bias(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
                               const int* block_table, int max_blocks, const int* token_seq, const int* positions, void* out,
                               int ld_out, int n_tokens, int n_heads, int n_kv_heads, int head_dim, int page_size, float scale,
                               int window, float softcap, int chunk, int num_pages, int dtype, const float* sink,
                               const float* out_gate, const float* dist_bias, int n_dist, int* status, cudaStream_t stream);
int sandy_prefill_attention_bias(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
                                 const int* block_table, int max_blocks, const int* q_start, const int* kv_before, void* out,
                                 int ld_out, int n_seqs, int max_q_len, int n_heads, int n_kv_heads, int head_dim,
                                 int page_size, float scale, int window, float softcap, int chunk, int num_pages,
                                 const float* sink, const float* out_gate, const float* dist_bias, int n_dist, int* status,
                                 cudaStream_t stream);
int sandy_decode_attention_shared_bias(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
                                       const int* block_table, int max_blocks, const int* token_seq, const int* positions,
                                       void* out, int ld_out, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                       int page_size, float scale, int window, float softcap, int chunk, int splits,
                                       int num_pages, const float* sink, const float* out_gate, const float* dist_bias,
                                       int n_dist, float* scratch, int* status, cudaStream_t stream);
int sandy_prefill_attention_cap(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
                                const int* block_table, int max_blocks, const int* q_start, const int* kv_before, void* out,
                                int ld_out, int n_seqs, int max_q_len, int n_heads, int n_kv_heads, int head_dim,
                                int page_size, float scale, int window, float softcap, int chunk, int num_pages,
                                const float* sink, const float* out_gate, int* status, cudaStream_t stream);
int sandy_decode_attention_shared_cap(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
                                      const int* block_table, int max_blocks, const int* token_seq, const int* positions,
                                      void* out, int ld_out, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                      int page_size, float scale, int window, float softcap, int chunk, int splits,
                                      int num_pages, const float* sink, const float* out_gate, float* scratch, int* status,
                                      cudaStream_t stream);
int sandy_decode_attention_cluster_ext(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
                                       const int* block_table, int max_blocks, const int* token_seq, const int* positions,
                                       void* out, int ld_out, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                       int page_size, float scale, int window, int num_splits, int num_pages, int dtype,
                                       const float* sink, const float* out_gate, int* status, cudaStream_t stream);
int sandy_decode_attention_ext(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
                               const int* block_table, int max_blocks, const int* token_seq, const int* positions, void* out,
                               int ld_out, float* scratch, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                               int page_size, float scale, int window, int num_splits, int num_pages, int dtype,
                               const float* sink, const float* out_gate, int* status, cudaStream_t stream);
int sandy_decode_attention_mma_ext(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
                                   const int* block_table, int max_blocks, const int* token_seq, const int* positions,
                                   void* out, int ld_out, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                   int page_size, float scale, int window, int num_splits, int num_pages, int max_keys,
                                   const float* sink, const float* out_gate, int* status, cudaStream_t stream);
int sandy_decode_attention_bulk_ext(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
                                    const int* block_table, int max_blocks, const int* token_seq, const int* positions,
                                    void* out, int ld_out, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                    int page_size, float scale, int window, int num_splits, int num_pages, int dtype,
                                    const float* sink, const float* out_gate, int* status, cudaStream_t stream);
int sandy_prefill_attention_ext(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
                                const int* block_table, int max_blocks, const int* q_start, const int* kv_before, void* out,
                                int ld_out, int n_seqs, int max_q_len, int n_heads, int n_kv_heads, int head_dim,
                                int page_size, float scale, int window, int num_pages, const float* sink,
                                const float* out_gate, int* status, cudaStream_t stream);
int sandy_prefill_attention_tc_ext(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
                                   const int* block_table, int max_blocks, const int* q_start, const int* kv_before,
                                   void* out, int ld_out, int n_seqs, int max_q_len, int n_heads, int n_kv_heads,
                                   int head_dim, int page_size, float scale, int window, int num_pages, const float* sink,
                                   const float* out_gate, int* status, cudaStream_t stream);
int sandy_prefill_attention_tc_cap(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
                                   const int* block_table, int max_blocks, const int* q_start, const int* kv_before,
                                   void* out, int ld_out, int n_seqs, int max_q_len, int n_heads, int n_kv_heads,
                                   int head_dim, int page_size, float scale, int window, float softcap, int chunk,
                                   int num_pages, const float* sink, const float* out_gate, int* status, cudaStream_t stream);

/* attention_decode_shared.cu */
long long sandy_decode_attention_shared_scratch(int n_tokens, int n_heads, int n_kv_heads, int head_dim, int splits);
int sandy_decode_attention_shared(const void* q, int ld_q, const void* k_cache, const void* v_cache, long long page_stride,
                                  const int* block_table, int max_blocks, const int* token_seq, const int* positions, void* out,
                                  int ld_out, int n_tokens, int n_heads, int n_kv_heads, int head_dim, int page_size, float scale,
                                  int window, int splits, int num_pages, const float* sink, const float* out_gate, float* scratch,
                                  int* status, cudaStream_t stream);

/* attention_prepare.cu */
int sandy_attention_prepare(const void* proj, int ld, int q_off, int k_off, int v_off, int n_tokens, int n_heads,
                            int n_kv_heads, int qk_dim, int v_dim, int pad_dim, const float* q_gain, const float* k_gain,
                            float eps, const float* freq, int rot_dims, const int* positions, const int* token_seq,
                            const int* block_table, int max_blocks, void* k_cache, void* v_cache, long long page_stride,
                            int page_size, int num_pages, int write_cache, void* q_out, int ld_q, const float* gate_in,
                            int ld_gate, float* gate_out, float gate_scale, int dtype, int* status, cudaStream_t stream);

int sandy_attention_prepare_ext(const void* proj, int ld, int q_off, int k_off, int v_off, int n_tokens, int n_heads,
                                int n_kv_heads, int qk_dim, int v_dim, int pad_dim, const float* q_gain, const float* k_gain,
                                float eps, const float* freq, int rot_dims, const int* positions, const int* token_seq,
                                const int* block_table, int max_blocks, void* k_cache, void* v_cache, long long page_stride,
                                int page_size, int num_pages, int write_cache, void* q_out, int ld_q, const float* gate_in,
                                int ld_gate, float* gate_out, float gate_scale, const float* q_head_scale, float v_unit_eps,
                                int dtype, int* status, cudaStream_t stream);

/* ... with every query and key head over its own root mean square (per_head_norm) and a factor on the query that grows
   with the position, 1 + q_pos_coef * ln(floor((p + 1) / q_pos_every) + 1) (q_pos_every 0: none). */
int sandy_attention_prepare_pos(const void* proj, int ld, int q_off, int k_off, int v_off, int n_tokens, int n_heads,
                                int n_kv_heads, int qk_dim, int v_dim, int pad_dim, const float* q_gain, const float* k_gain,
                                float eps, const float* freq, int rot_dims, const int* positions, const int* token_seq,
                                const int* block_table, int max_blocks, void* k_cache, void* v_cache, long long page_stride,
                                int page_size, int num_pages, int write_cache, void* q_out, int ld_q, const float* gate_in,
                                int ld_gate, float* gate_out, float gate_scale, const float* q_head_scale, float v_unit_eps,
                                int per_head_norm, float q_pos_coef, int q_pos_every, int dtype, int* status,
                                cudaStream_t stream);

/* rmsnorm.cu */
int sandy_rmsnorm_shift(const float* x, int ldx, const float* gain, const float* mix, float* state, long long state_stride,
                        const int* token_seq, const int* q_start, const int* seq_slots, void* out, int ldo, int n_tokens,
                        int width, float eps, int out_dtype, cudaStream_t stream);
int sandy_rmsnorm_keep(const float* x, int ldx, const float* gain, float* state, long long state_stride, const int* q_start,
                       const int* seq_slots, int n_seqs, int width, float eps, cudaStream_t stream);
int sandy_rmsnorm(const float* x, int ldx, const float* gain, void* out, int ldo, const int* rows, int n_rows, int width,
                  float eps, int out_dtype, cudaStream_t stream);
int sandy_rmsnorm_add(const float* y, int ldy, const float* gain, float* x, int ldx, int n_rows, int width, float eps,
                      float mult, cudaStream_t stream);
int sandy_head_norm_gate(const float* o, int ldo, const float* gain, int gain_stride, const void* gate, int ldg,
                         int gate_dtype, void* out, int ld_out, int out_dtype, int n_tokens, int n_heads, int dim, float eps,
                         int act, float scale, cudaStream_t stream);

/* elementwise.cu */
int sandy_glu(const void* a, const void* b, int ld_in, void* out, int ld_out, int rows, int cols, int act, int dtype,
              cudaStream_t stream);
int sandy_cast_cols(const float* x, int ldx, void* out, int ld_out, int rows, int cols, int out_dtype, cudaStream_t stream);
int sandy_scale_add(const float* y, int ldy, const float* gain, const float* y2, int ldy2, const float* gain2, float* x, int ldx,
                    int rows, int cols, cudaStream_t stream);
int sandy_scale_f32(float* x, long long n, float s, cudaStream_t stream);
int sandy_glu_clamped(const void* a, const void* b, int ld_in, void* out, int ld_out, int rows, int cols, float limit,
                      float alpha, int dtype, cudaStream_t stream);
int sandy_stream_add(float* x, int ldx, const float* x0, int ldx0, const float* row, int rows, int cols, cudaStream_t stream);
int sandy_softcap_f32(float* x, long long n, float cap, cudaStream_t stream);

/* latent_prepare.cu */
int sandy_latent_prepare(const float* down, int ld_down, int n_tokens, int q_rank, int kv_rank, int rot_dim, const float* q_gain,
                         const float* kv_gain, float eps, const float* freq, int rot_dims, const int* positions,
                         const int* token_seq, const int* block_table, int max_blocks, void* cache, long long page_stride,
                         int page_size, int num_pages, int pad_dim, int write_cache, void* q_latent, int ld_ql, const void* q,
                         int ld_q, int n_heads, int qk_dim, void* q_abs, int ld_qa, int dtype, int* status, cudaStream_t stream);

/* grouped_gemm.cu */
int sandy_head_product(const void* a, int lda, int a_gcols, const void* w, long long w_gstride, int ldw, void* out, int ldo,
                       int o_gcols, int rows, int n_groups, int N, int K, int in_dtype, int out_dtype, cudaStream_t stream);
int sandy_expert_product(const void* a, int lda, const void* w, long long w_gstride, int ldw, void* out, int ldo, int n_slots,
                         int n_groups, int N, int K, const int* group_start, const int* a_row, int a_row_div, int act,
                         int in_dtype, int out_dtype, cudaStream_t stream);

/* grouped_gemm_tc.cu */
int sandy_expert_product_tc(const void* a, int lda, const void* w, int ldw, void* out, int ldo, int n_slots, int n_groups, int N,
                            int K, const int* group_start, int act, int out_dtype, int* status, cudaStream_t stream);

/* moe.cu */
int sandy_moe_route(const float* logits, int ld, const float* bias, int n_tokens, int n_experts, int top, int* expert_of,
                    float* weight_of, cudaStream_t stream);
int sandy_moe_route_scored(const float* logits, int ld, const float* correction, int n_tokens, int n_experts, int top,
                           int n_groups, int keep_groups, int group_rank, float weight_scale, float norm_eps, int* expert_of,
                           float* weight_of, cudaStream_t stream);
int sandy_moe_group(const int* expert_of, int n_entries, int n_experts, int* group_start, int* entry_of_slot, int* slot_of_entry,
                    cudaStream_t stream);
int sandy_moe_gather(const void* x, long long pitch_x, const int* entry_of_slot, int top, void* out, long long pitch_out, int n_slots,
                     int bytes_per_row, cudaStream_t stream);
int sandy_moe_combine(const float* rows, int ld_rows, const float* weight_of, const int* slot_of_entry, int n_tokens, int top,
                      float* y, int ldy, int width, int add, cudaStream_t stream);

int sandy_moe_route_softmax(const float* logits, int ld, const float* correction, int n_tokens, int n_experts, int top,
                            float weight_scale, float norm_eps, int renormalize, int* expert_of, float* weight_of,
                            cudaStream_t stream);
int sandy_moe_combine_identity(const float* rows, int ld_rows, const float* weight_of, const int* slot_of_entry,
                               const int* expert_of, int n_real, const void* h, int ldh, int h_dtype, int n_tokens, int top,
                               float* y, int ldy, int width, int add, cudaStream_t stream);

/* streams.cu */
int sandy_streams_step(float* X, int ldX, int n_tokens, int n_streams, int width, const float* y, int ldy, const float* gate,
                       int ldg, const float* gate_bias, const float* mix, const float* out_w, const float* in_w,
                       const float* gain, float eps, void* h, int ldh, int h_dtype, float* sum_out, int ld_sum,
                       cudaStream_t stream);
int sandy_streams_step_conv(float* X, int ldX, int n_tokens, int n_streams, int width, const float* y, int ldy, const float* gate,
                            int ldg, const float* gate_bias, const float* mix, const float* out_w, const float* in_w,
                            const float* gain, float eps, void* h, int ldh, int h_dtype, float* sum_out, int ld_sum,
                            const float* taps, int n_taps, float* state, long long state_stride, long long tail_off,
                            const int* token_seq, const int* seq_slots, void* c, int ldc, cudaStream_t stream);
int sandy_streams_max(void);
int sandy_streams_spread(const float* x, int ldx, float* X, int ldX, int n_tokens, int n_streams, int width, cudaStream_t stream);
int sandy_canon_conv(const void* h, int ldh, const float* taps, int n_taps, const float* state, long long state_stride,
                     long long tail_off, const int* token_seq, const int* q_start, const int* seq_slots, void* c, int ldc,
                     int n_tokens, int width, int dtype, cudaStream_t stream);
int sandy_embed_bigram(const int* ids, const int* positions, const int* token_seq, const int* q_start, const int* seq_slots,
                       const void* wte, const void* bigram, const void* wpe, int buckets, long long mul_prev, long long mul_cur,
                       int* state, long long state_stride, float* x, int ldx, int n_tokens, int vocab, int n_pos, int width,
                       int table_dtype, int keep, int* status, cudaStream_t stream);
int sandy_bigram_keep(const int* ids, const int* q_start, const int* seq_slots, int* state, long long state_stride, int n_seqs,
                      cudaStream_t stream);

/* ssm_state.cu */
long long sandy_ssm_state_floats(int n_heads, int state, int v_dim);
int sandy_ssm_prepare(const void* proj, int ld, int dtype, int channels, const float* taps, int n_taps, const float* conv_bias,
                      const float* dt_raw, int ld_dt, const float* dt_bias, const float* a_log, int n_heads, float* state,
                      long long state_stride, long long tail_off, const int* token_seq, const int* q_start, const int* seq_slots,
                      float* xbc, int ld_xbc, float* dta, int n_tokens, int keep, cudaStream_t stream);
int sandy_ssm_scan(const float* xbc, int ld, const float* dta, const float* d_skip, float* state, long long state_stride,
                   const int* q_start, const int* seq_slots, float* out, int ld_out, int n_seqs, int n_heads, int n_groups,
                   int state_dim, int v_dim, cudaStream_t stream);
int sandy_gated_group_norm(const float* y, int ldy, const void* z, int ldz, const float* gain, float eps, int groups, void* out,
                           int ld_out, int n_tokens, int cols, int dtype, cudaStream_t stream);

/* matrix_state.cu */
long long sandy_mlstm_state_floats(int n_heads, int qk_dim, int v_dim);
int sandy_delta_prepare(const void* proj, int ld, int dtype, const float* taps, int n_taps, const float* gates, int ld_gates,
                        const float* a_log, const float* dt_bias, const float* state, long long state_stride,
                        long long tail_off, const int* token_seq, const int* q_start, const int* seq_slots, float* qkv,
                        int ld_qkv, float* bg, int n_tokens, int n_heads, int n_qk_heads, int qk_dim, int v_dim,
                        float q_scale, cudaStream_t stream);
int sandy_conv_tail(const void* proj, int ld, int dtype, int channels, int n_taps, float* state, long long state_stride,
                    long long tail_off, const int* q_start, const int* seq_slots, int n_seqs, cudaStream_t stream);
int sandy_delta_scan(const float* qkv, int ld, const float* bg, float* state, long long state_stride, const int* q_start,
                     const int* seq_slots, float* out, int ld_out, int n_seqs, int n_heads, int n_qk_heads, int qk_dim,
                     int v_dim, int long_from, cudaStream_t stream);
int sandy_delta_chunk_scan(const float* qkv, int ld, const float* bg, float* state, long long state_stride,
                           const int* q_start, const int* seq_slots, float* out, int ld_out, int n_seqs, int n_heads,
                           int n_qk_heads, int qk_dim, int v_dim, int long_from, cudaStream_t stream);
int sandy_mlstm_scan(const void* proj, int ld, int dtype, int q_off, int k_off, int v_off, const float* gates, int ld_gates,
                     const float* gate_bias, float cap, float q_scale, float* state, long long state_stride,
                     const int* q_start, const int* seq_slots, float* out, int ld_out, int n_seqs, int n_heads, int qk_dim,
                     int v_dim, int long_from, cudaStream_t stream);
int sandy_mlstm_chunk_scan(const void* proj, int ld, int dtype, int q_off, int k_off, int v_off, const float* gates,
                           int ld_gates, const float* gate_bias, float cap, float q_scale, float* state,
                           long long state_stride, const int* q_start, const int* seq_slots, float* out, int ld_out,
                           int n_seqs, int n_heads, int qk_dim, int v_dim, int long_from, cudaStream_t stream);

/* sampling.cu */
int sandy_sample(const float* logits, int ld, int n_rows, int vocab, const float* temperature, const int* top_k,
                 const float* top_p, const float* uniform, int* out_token, int* status, int* token_ids,
                 const int* logit_rows, int* positions, int* out_tokens, int* row_step, cudaStream_t stream);

#ifdef __cplusplus
}
#endif

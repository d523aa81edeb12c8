// The C interface of the janas_b200 kernel library.
//
// Every function takes device pointers and the stream to launch on, allocates
// nothing and returns 0 or a negative code (JB_EINVAL: a size or type the
// kernel does not take; JB_ELAUNCH: the launch failed).  The Python side
// (janas_b200/csrc/ops.py) checks shapes and types before it calls in here.
//
// The kernels are launched so that their CTAs may start while the kernel before
// them in the stream still runs, and they read what cannot depend on it before
// they wait for it: weights, norm weights, rotation tables, and the index arrays
// row_pos, row_seq and block_table.  None of these may be the output of another of
// this library's kernels launched just before (a copy, or any kernel launched in
// the ordinary way, is fine: nothing starts before those have finished).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

// element types of buffers
#define JB_F32 0
#define JB_BF16 1

// activations of jb_activation
#define JB_ACT_RELU2 0
#define JB_ACT_RELU 1
#define JB_ACT_GELU_TANH 2
#define JB_ACT_SILU 3
// modes of jb_qkv_prepare_append: the rotation turns neighbours (2i, 2i + 1) instead of (i, i + half);
// q and k heads are divided by their root mean square after the rotation
#define JB_ROT_PAIRS 1
#define JB_UNIT_NORM 2

#ifdef __cplusplus
extern "C" {
#endif

int jb_page(void);
int jb_embed(const void *table, int table_dt, const int32_t *tokens, float *x, int n, int dm,
             cudaStream_t st);
int jb_rmsnorm(float *x, const float *delta, int S, long long delta_stride,
               const int32_t *row_idx, const void *w, int w_dt, void *out, int out_dt, int n_out,
               int dm, float eps, cudaStream_t st);
int jb_swiglu(const float *gu, int S, long long stride, void *out, int out_dt, int n, int ff,
              cudaStream_t st);
int jb_rope_table(float *cs, float *sn, const float *inv_freq, int n_pos, int half,
                  cudaStream_t st);
int jb_qk_norm_rope_append(const float *qkv, int S, long long split_stride, const void *q_w,
                           const void *k_w, int w_dt, float eps, const float *cs, const float *sn,
                           int rot_half, const int32_t *row_pos, const int32_t *row_seq,
                           const int32_t *block_table, int bt_stride, void *q_out, void *k_cache,
                           void *v_cache, int cache_dt, int n, int nh, int nkv, int hd,
                           cudaStream_t st);
int jb_attention_chunk(void);
long long jb_attention_scratch(int n_rows, int nh, int hd, int max_chunks);
int jb_attention(const void *q, const void *k_cache, const void *v_cache, int dt,
                 const int32_t *row_pos, const int32_t *row_seq, const int32_t *block_table,
                 int bt_stride, float *scratch, void *out, int row0, int n_rows, int nh, int nkv,
                 int hd, int window, float scale, int max_chunks, cudaStream_t st);
int jb_attention_merge(const float *scratch, const int32_t *row_pos, void *out, int dt, int row0,
                       int n_rows, int nh, int hd, int window, int max_parts, int chunks_per_part,
                       cudaStream_t st);
int jb_attention_sink(const void *q, const void *k_cache, const void *v_cache, int dt,
                      const int32_t *row_pos, const int32_t *row_seq, const int32_t *block_table,
                      int bt_stride, float *scratch, void *out, int row0, int n_rows, int nh,
                      int nkv, int hd, int vd, int window, float scale, const float *head_scale,
                      const float *sink, int max_chunks, cudaStream_t st);
int jb_attention_merge_sink(const float *scratch, const int32_t *row_pos, void *out, int dt,
                            int row0, int n_rows, int nh, int hd, int window, int max_parts,
                            int chunks_per_part, const float *sink, cudaStream_t st);
int jb_embed_pos(const void *table, int table_dt, const void *pos_table, int pos_dt,
                 const int32_t *tokens, const int32_t *row_pos, float *x, int n, int dm,
                 cudaStream_t st);
int jb_dyt(float *x, const float *delta, int S, long long delta_stride, const int32_t *row_idx,
           const float *w, const float *b, const float *alpha, void *out, int out_dt, int n_out,
           int dm, cudaStream_t st);
int jb_gate_mul(const float *y, int Sy, long long y_stride, const float *y_bias, const float *g,
                int Sg, long long g_stride, int g_ld, int g_col0, const float *g_bias, float *out,
                int n, int dm, cudaStream_t st);
int jb_gated_dyt_residual(float *x, const float *y, int Sy, long long y_stride,
                          const float *y_bias, const float *g, int Sg, long long g_stride,
                          int g_ld, int g_col0, const float *g_bias, const float *pw,
                          const float *pb, const float *palpha, const float *nw, const float *nb,
                          const float *nalpha, void *out, int out_dt, int n, int dm, int fast,
                          cudaStream_t st);
int jb_polynorm(const float *z, int S, long long stride, int z_ld, const float *coef, float eps,
                void *out, int out_dt, int n, int ff, cudaStream_t st);
int jb_scale(float *x, float s, long long total, cudaStream_t st);
int jb_add_bias(float *y, const float *bias, int n, int m, cudaStream_t st);
int jb_qkv_bias_append(const float *qkv, int S, long long stride, int ld, const float *bias,
                       const int32_t *row_pos, const int32_t *row_seq, const int32_t *block_table,
                       int bt_stride, void *q_out, void *k_cache, void *v_cache, int cache_dt,
                       int n, int nh, int nkv, int hd, int vd, int append, cudaStream_t st);
int jb_qkv_bias_append_temp(const float *qkv, int S, long long stride, int ld, const float *bias,
                            const int32_t *row_pos, const int32_t *row_seq,
                            const int32_t *block_table, int bt_stride, void *q_out, void *k_cache,
                            void *v_cache, int cache_dt, int n, int nh, int nkv, int hd, int vd,
                            int append, float q_coef, int q_every, cudaStream_t st);
int jb_attention_ext(const void *q, const void *k_cache, const void *v_cache, int dt,
                     const int32_t *row_pos, const int32_t *row_seq, const int32_t *block_table,
                     int bt_stride, float *scratch, void *out, int row0, int n_rows, int nh,
                     int nkv, int hd, int vd, int window, float scale, const float *head_scale,
                     const float *sink, int max_chunks, int v_ld, float softcap,
                     const float *slopes, long long head_major_rows, cudaStream_t st);
int jb_attention_kept_chunks(int window, int keep_first);
int jb_attention_gen(const void *q, const void *k_cache, const void *v_cache, int dt,
                     const int32_t *row_pos, const int32_t *row_seq, const int32_t *block_table,
                     int bt_stride, float *scratch, void *out, int row0, int n_rows, int nh,
                     int nkv, int hd, int vd, int window, float scale, const float *head_scale,
                     const float *sink, int max_chunks, int v_ld, float softcap,
                     const float *slopes, long long head_major_rows, int keep_first,
                     const float *score_bias, cudaStream_t st);
int jb_layernorm(float *x, const float *a, int Sa, long long a_stride, const float *b, int Sb,
                 long long b_stride, float mult, const int32_t *row_idx, const float *w,
                 const float *bias, void *out, int out_dt, int n_out, int dm, float eps,
                 cudaStream_t st);
int jb_latent_down(const float *P, int S, long long stride, int ld, int q_col0, int q_rank,
                   const float *wq, int kv_col0, int kv_rank, const float *wkv, int rot_dim,
                   const float *cs, const float *sn, int rot_half, const int32_t *row_pos,
                   const int32_t *row_seq, const int32_t *block_table, int bt_stride, void *cq_out,
                   void *k_cache, int cache_dt, int n, float eps, cudaStream_t st);
int jb_latent_down_rows(const float *P, int S, long long stride, int ld, int q_col0, int q_rank,
                        const float *wq, int kv_col0, int kv_rank, const float *wkv, int rot_dim,
                        const float *cs, const float *sn, int rot_half, const int32_t *row_pos,
                        const int32_t *row_seq, const int32_t *block_table, int bt_stride,
                        void *cq_out, void *k_cache, void *rows_out, int cache_dt, int n, float eps,
                        cudaStream_t st);
int jb_gate_rows(const void *a, const float *g, int Sg, long long g_stride, int g_ld, int g_col0,
                 void *out, int dt, int n, int width, cudaStream_t st);
int jb_latent_q_split(const float *Q, int S, long long stride, int nh, int D, int R, int C,
                      const float *cs, const float *sn, int rot_half, const int32_t *row_pos,
                      void *q_plain, void *q_lat, int dt, int n, cudaStream_t st);
int jb_latent_q_join(const float *A, int S, int nh, int C, int R, void *q_lat, int dt, int n,
                     cudaStream_t st);
int jb_heads_gate(const float *A, int S, int nh, int Dv, const float *g, int Sg, long long g_stride,
                  int g_ld, int g_col0, void *out, int out_dt, int n, cudaStream_t st);
int jb_transpose_heads(const void *in, void *out, int dt, int H, int D, int C, cudaStream_t st);
int jb_activation(const float *z, int S, long long stride, int ld, int kind, void *out, int out_dt,
                  int n, int ff, cudaStream_t st);
int jb_qkv_prepare_append(const float *qkv, int S, long long split_stride, int ld, const float *bias,
                          const float *q_w, const float *k_w, float eps, const float *cs,
                          const float *sn, int rot_half, const int32_t *row_pos,
                          const int32_t *row_seq, const int32_t *block_table, int bt_stride,
                          void *q_out, void *k_cache, void *v_cache, int cache_dt, int n, int nh,
                          int nkv, int hd, int vd, int mode, cudaStream_t st);
int jb_norm_residual(float *x, const float *a, int Sa, long long a_stride, const float *a_bias,
                     const void *skip, int skip_dt, const float *coef, int coef_ld, const float *w,
                     const float *bias, int n, int dm, float eps, int rms, int few_rows,
                     cudaStream_t st);
int jb_short_conv(const float *x, const float *w, float *state, long long slot_stride, const int32_t *row_pos,
                  const int32_t *row_seq, const int32_t *seq_slot, void *out, int out_dt, int n,
                  int dm, int taps, int what, cudaStream_t st);
int jb_mingru_piece(void);
long long jb_mingru_scratch(int n, int n_seqs, int W, int every_row_starts);
int jb_mingru(const float *P, int S, long long stride, int ld, int col0, const float *bias,
              float *state, const int32_t *row_seq, const int32_t *seq_slot, float *scratch,
              void *out, int out_dt, int n, int n_seqs, int W, int every_row_starts,
              cudaStream_t st);
int jb_moe_route(const float *P, int S, long long stride, int ld, int col0, const float *correction,
                 float *weights, float *skip_coef, int n, int E, int groups, int keep, int top,
                 int first_identity, float scale, int sigmoid_scores, int group_best, cudaStream_t st);
int jb_gated_weighted(const float *z, int S, long long stride, int ld, const float *weights, int w_ld,
                      int n_experts, int ff, int kind, void *out, int out_dt, int n, cudaStream_t st);
int jb_causal_conv(const float *u, int S, long long stride, int ld, int col0, const float *w,
                   const float *bias, float *state, long long slot_stride, const int32_t *row_pos,
                   const int32_t *row_seq, const int32_t *seq_slot, void *out, int out_dt, int out_ld,
                   int n, int C, int taps, int act, int what, cudaStream_t st);
int jb_matrix_state_scan(const float *src, int S, long long stride, int ld, int val_col0, int key_col0,
                         int qry_col0, int silu, const float *dt, int dt_S, long long dt_stride,
                         int dt_ld, int dt_col0, const float *dt_bias, const float *a_log,
                         const float *skip, const float *decay, float *state, long long slot_stride,
                         const int32_t *row_seq, const int32_t *seq_slot, float *y, int n, int n_seqs,
                         int H, int G, int N, int P, int every_row_starts, float *scratch, int max_len,
                         cudaStream_t st);
int jb_matrix_state_piece(void);
long long jb_matrix_state_scratch(int n_seqs, int max_len, int H, int N, int P);
int jb_gated_part_norm(const float *y, const float *pre, int pre_S, long long pre_stride, int pre_ld,
                       int pre_col0, const float *post, int post_S, long long post_stride, int post_ld,
                       int post_col0, const float *w, float eps, void *out, int out_dt, int n, int width,
                       int parts, int few_rows, cudaStream_t st);
int jb_pair_combine(const float *L, int SL, long long strideL, const float *R, int SR, long long strideR,
                    const float *wl, const float *wr, float sl, float sr, float eps, float *out, int n,
                    int m, int few_rows, cudaStream_t st);
int jb_token_gate(const float *P, int S, long long stride, int ld, const void *table, int table_dt,
                  int table_ld, int col0, const int32_t *tokens, void *out, int out_dt, int n, int dim,
                  cudaStream_t st);
int jb_activation_weighted(const float *z, int S, long long stride, int ld, const float *weights,
                           int w_ld, int n_experts, int ff, int kind, void *out, int out_dt, int n,
                           int width, cudaStream_t st);
int jb_add_row_scaled(float *y, const void *skip, int skip_dt, const float *coef, int coef_ld, int n, int m,
                      cudaStream_t st);
int jb_attn_tc_decode_runs(int nh, int nkv, int hd);
int jb_attn_tc_ok(int nh, int nkv, int hd);
int jb_attn_tc_block_positions(int nh, int nkv);
int jb_attn_tc_prefill(const void *q, const void *k_cache, const void *v_cache, long long n_pages,
                       const int32_t *qblk, int n_blocks, const int32_t *block_table,
                       int bt_stride, void *out, int n, int nh, int nkv, int hd, int window,
                       float scale, cudaStream_t st);
int jb_attn_tc_decode(const void *q, const void *k_cache, const void *v_cache, long long n_pages,
                      const int32_t *row_pos, const int32_t *row_seq, const int32_t *block_table,
                      int bt_stride, float *part, int n, int row0, int n_rows, int nh, int nkv,
                      int hd, int window, float scale, int max_chunks, int chunks_per_cta,
                      cudaStream_t st);
int jb_attn_tc_decode_qkv(const float *qkv, int S, long long split_stride, const void *q_w,
                          const void *k_w, int w_dt, float eps, const float *cs, const float *sn,
                          void *k_cache, void *v_cache, int append, long long n_pages,
                          const int32_t *row_pos, const int32_t *row_seq,
                          const int32_t *block_table, int bt_stride, float *part, int n, int row0,
                          int n_rows, int nh, int nkv, int hd, int window, float scale,
                          int max_chunks, int chunks_per_cta, cudaStream_t st);
int jb_attn_tc_prefill_sink(const void *q, const void *k_cache, const void *v_cache,
                            long long n_pages, const int32_t *qblk, int n_blocks,
                            const int32_t *block_table, int bt_stride, void *out, int n, int nh,
                            int nkv, int hd, int window, float scale, const float *head_scale,
                            const float *sink, cudaStream_t st);
int jb_attn_tc_decode_scaled(const void *q, const void *k_cache, const void *v_cache,
                             long long n_pages, const int32_t *row_pos, const int32_t *row_seq,
                             const int32_t *block_table, int bt_stride, float *part, int n,
                             int row0, int n_rows, int nh, int nkv, int hd, int window,
                             float scale, const float *head_scale, int max_chunks,
                             int chunks_per_cta, cudaStream_t st);
int jb_attn_tc_decode_qkv_bias(const float *qkv, int S, long long split_stride, const float *bias,
                               const void *q_w, const void *k_w, int w_dt, float eps,
                               const float *cs, const float *sn, void *k_cache, void *v_cache,
                               int append, long long n_pages, const int32_t *row_pos,
                               const int32_t *row_seq, const int32_t *block_table, int bt_stride,
                               float *part, int n, int row0, int n_rows, int nh, int nkv, int hd,
                               int window, float scale, const float *head_scale, long long ld,
                               int max_chunks, int chunks_per_cta, cudaStream_t st);
int jb_attn_tc_prefill_ext(const void *q, const void *k_cache, const void *v_cache,
                           long long n_pages, const int32_t *qblk, int n_blocks,
                           const int32_t *block_table, int bt_stride, void *out, int n, int nh,
                           int nkv, int hd, int window, float scale, const float *head_scale,
                           const float *sink, float softcap, const float *slopes, cudaStream_t st);
int jb_attn_tc_decode_ext(const void *q, const void *k_cache, const void *v_cache,
                          long long n_pages, const int32_t *row_pos, const int32_t *row_seq,
                          const int32_t *block_table, int bt_stride, float *part, int n, int row0,
                          int n_rows, int nh, int nkv, int hd, int window, float scale,
                          const float *head_scale, float softcap, const float *slopes,
                          int max_chunks, int chunks_per_cta, cudaStream_t st);
int jb_attn_tc_prefill_gen(const void *q, const void *k_cache, const void *v_cache,
                           long long n_pages, const int32_t *qblk, int n_blocks,
                           const int32_t *block_table, int bt_stride, void *out, int n, int nh,
                           int nkv, int hd, int window, float scale, const float *head_scale,
                           const float *sink, float softcap, const float *slopes, int keep_first,
                           const float *score_bias, cudaStream_t st);
int jb_attn_tc_decode_gen(const void *q, const void *k_cache, const void *v_cache,
                          long long n_pages, const int32_t *row_pos, const int32_t *row_seq,
                          const int32_t *block_table, int bt_stride, float *part, int n, int row0,
                          int n_rows, int nh, int nkv, int hd, int window, float scale,
                          const float *head_scale, float softcap, const float *slopes,
                          int keep_first, const float *score_bias, int max_chunks,
                          int chunks_per_cta, cudaStream_t st);
int jb_attention_merge_gen(const float *scratch, const int32_t *row_pos, void *out, int dt,
                           int row0, int n_rows, int nh, int hd, int window, int max_parts,
                           int chunks_per_part, const float *sink, int keep_first, int plain_sum,
                           cudaStream_t st);
int jb_attn_tc_error(void);
long long jb_gemm_simt_scratch(int n, int m, int k);
int jb_gemm_simt(const void *A, int a_dt, const void *W, int w_dt, float *out, int n, int m, int k,
                 float *scratch, cudaStream_t st);
int jb_gemm_tc_ok(const void *A, const void *W, int n, int m, int k);
int jb_gemm_tc_splits(int n, int m, int k);
int jb_gemm_tc(const void *A, const void *W, float *out, int n, int m, int k, int splits,
               cudaStream_t st);
int jb_gemm_tc_heads(const void *A, const void *W, float *out, int n, int m, int k, int splits,
                     int heads, cudaStream_t st);
int jb_gemm_tc_swiglu(const void *A, const void *W, void *out_act, int n, int ff, int k,
                      cudaStream_t st);
int jb_gemm_tc_error(void);
int jb_gemm_tc_force_tile(int tokens);
int jb_gemm_tc_last_tile(void);
int jb_wait_selftest(long long limit_cycles);
int jb_sample_small_cap(void);
int jb_sample_needs_big(int V, int top_k);
int jb_sampler_set(const int32_t *slots, int n, const unsigned long long *seeds,
                   const float *temperature, const int32_t *top_k, const float *top_p,
                   const float *min_p, unsigned long long *rng_out, float *temperature_out,
                   int32_t *top_k_out, float *top_p_out, float *min_p_out, cudaStream_t st);
long long jb_sample_scratch(int rows, int V);
int jb_sample_launches(int V, long long big_cap, int sampled);
int jb_sample(const float *logits, int rows, int V, const int32_t *row_slot,
              const float *temperature, const int32_t *top_k, const float *top_p,
              const float *min_p, unsigned long long *rng, unsigned long long *big_keys,
              float *big_probs, long long big_cap, unsigned long long *chunk_keys, int32_t *out,
              int32_t *forced, cudaStream_t st);

#ifdef __cplusplus
}
#endif

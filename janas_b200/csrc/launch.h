// The kernels as checked C++ calls over device memory.
//
// Each function takes what the kernel takes, gets its output and scratch from
// the device's pool of temporaries, launches on the device's stream and throws a
// jb::Error when the kernel library refuses the sizes (JB_LLM_EINVAL) or the
// launch fails (JB_LLM_EFAIL).  There is no CPU fallback and no library model
// code behind these functions.
//
// Conventions: the residual stream and every matrix product's output are
// float32.  A product's output is a stack [S, n, m] of S partial sums whose sum
// over S is the result (S = 1 unless the product was split over k); the kernels
// that consume a product add the partial sums in the order 0 .. S-1.
#pragma once

#include <cstdint>
#include <string>

#include "../engine/device.h"

namespace jb {

// float32 partial sums [S, n, m]
struct Stack {
    Buf buf;
    int S = 0;
    long long n = 0, m = 0;
    // float32 [m] on the device, still to be added once to every row of the sum (a
    // product's bias), or null.  The kernels that end a sublayer take it as it is;
    // for every other consumer resolve_bias() adds it into the first partial sum.
    const float *bias = nullptr;
    // Also still to be added: skip_coef[r * skip_coef_ld] * skip[r, :] for every row r (a
    // part's own input handed on with a weight per row: the identity experts of a routed
    // feed-forward).  skip: [n, m] of type skip_dt; null: nothing.  The kernel that ends a
    // sublayer with a norm on its result takes it; no other consumer does.
    const void *skip = nullptr;
    DType skip_dt = F32;
    const float *skip_coef = nullptr;
    long long skip_coef_ld = 1;
    Buf skip_hold;                      // keeps skip_coef's memory
    float *data() const { return (float *)buf.ptr; }
    long long stride() const { return n * m; }
    explicit operator bool() const { return S > 0; }
};

namespace ops {

// how many of the library's kernels have been launched (for measurements)
long long launches();
void count_launches(long long n);

int attention_chunk();
int sample_small_cap();
bool sample_needs_big(int vocab, int top_k);

// x[j, :] = table[tokens[j], :] as float32 [n, dm]; with a table of learned
// position vectors, plus pos_table[row_pos[j], :]
Buf embed(Device &d, const DevTensor &table, const int32_t *tokens, long long n,
          const DevTensor *pos_table = nullptr, const int32_t *row_pos = nullptr);

// The Dynamic Tanh norm's parameters on the device, all float32: w and b [dm], alpha [1].
struct DytParams {
    const float *w = nullptr, *b = nullptr, *alpha = nullptr;
};
// tanh(alpha x) w + b on the rows of x (float32 [n, dm]); delta and rows as in rmsnorm.
Buf dyt(Device &d, float *x, long long n, long long dm, const DytParams &p, DType out_dt,
        const Stack *delta, const int32_t *rows, long long n_out);
// (sum y + y.bias) * sigmoid(sum g + g_bias) as float32 [n, dm].  g's rows may be wider
// than dm: the gate is then its columns g_col0 .. g_col0 + dm - 1.  Biases: float32 [dm] or null.
Buf gate_mul(Device &d, const Stack &y, const Stack &g, long long g_col0, const float *g_bias);
// adds y.bias into y's first partial sum and clears it (nothing when there is none)
void resolve_bias(Device &d, Stack &y);
// x += dyt_post(gate_mul(...)) in place; with `next`, also returns dyt_next(x) in out_dt.
Buf gated_dyt_residual(Device &d, float *x, const Stack &y, const Stack &g, long long g_col0,
                       const float *g_bias, const DytParams &post, const DytParams *next, DType out_dt);
// c0 n(z) + c1 n(z^2) + c2 n(z^3) + c3 over the first ff columns of z's rows,
// n(u) = u / sqrt(mean(u^2) + eps); coef: float32 [4] on the device.  [n, ff] in out_dt.
Buf polynorm(Device &d, const Stack &z, long long ff, const float *coef, float eps, DType out_dt);
void scale_(Device &d, float *x, long long total, float s);

// Layer norm with weight and bias (float32 [dm] each; b may be null).
struct LnParams {
    const float *w = nullptr, *b = nullptr;
    float eps = 0.0f;
};
// (x - mean) / sqrt(var + eps) * w + b on the rows of x (float32 [n, dm]).  With a
// (and optionally b), two stacks of partial sums, x += mult * (sum a + sum b) happens
// first, in place.  rows as in rmsnorm (the add then runs as a launch of its own).
Buf layernorm(Device &d, float *x, long long n, long long dm, const LnParams &p, DType out_dt,
              const Stack *a, const Stack *b, float mult, const int32_t *rows, long long n_out);
// x += mult * (sum a + sum b) (b may be null)
void add_scaled_(Device &d, float *x, long long n, long long dm, const Stack &a, const Stack *b, float mult);

// act(sum z) over ff columns of z's rows, from col0 on; kind: "relu2" (the square of
// relu), "relu", "gelu_tanh", "silu".  [n, ff] in out_dt.
int activation_kind(const std::string &name);       // -1: unknown
Buf activation(Device &d, const Stack &z, long long ff, int kind, DType out_dt, long long col0 = 0);

// x += norm(sum y + y.bias + y's skip term) w (+ b): a norm on a sublayer's result alone,
// added to the residual stream in place.  rms: no mean is taken off.  few_rows: the
// bfloat16 path's kernel for a decode step's rows.
void norm_residual_(Device &d, float *x, const Stack &y, const LnParams &p, bool rms, bool few_rows);

// h = x + a causal convolution over time on every channel (w: float32 [dm, taps]), as
// [n, dm] in out_dt; state: float32 [taps - 1, dm] per slot, slot_stride floats apart (null
// with taps == 1).  write_h /
// write_state: what this launch does (see csrc/recurrent.cu for when both may be one).
Buf short_conv(Device &d, const float *x, long long n, long long dm, const float *w, int taps, float *state,
               long long slot_stride, const int32_t *row_pos, const int32_t *row_seq, const int32_t *seq_slot, DType out_dt,
               bool write_h, bool write_state);

// The minGRU's recurrence over the rows, from the sums P of [z | x | g] (columns col0 ..,
// W each; bias float32 [3 W] or null): S * silu(g) as [n, W] in out_dt; state: float32
// [slots, W], read and left updated.  every_row_starts: a decode step.
Buf mingru(Device &d, const Stack &P, long long col0, long long W, const float *bias, float *state,
           const int32_t *row_seq, const int32_t *seq_slot, int n_seqs, bool every_row_starts, DType out_dt);

// The router of a routed feed-forward (csrc/moe.cu): weights [n, E] float32 (0 for experts
// not chosen) and, with skip_coef, the summed weight of the chosen experts from
// first_identity on.
struct RouteParams {
    int experts = 0, groups = 1, keep = 1, top = 1, first_identity = 0;
    float scale = 1.0f;
    const float *correction = nullptr;
    bool sigmoid_scores = false;      // each score the sigmoid of its logit, instead of a softmax over all
    int group_best = 1;               // a group's score: the sum of this many of its largest choices
};
Buf moe_route(Device &d, const Stack &P, long long col0, const RouteParams &r, Buf *skip_coef);
// act(sum z) * weights[row, column / ff] over the first n_experts * ff columns of z, act
// alone over the rest up to width: [n, width] in out_dt.  weights: float32 [n, w_ld].
Buf activation_weighted(Device &d, const Stack &z, long long width, const float *weights, int w_ld, int n_experts,
                        long long ff, int kind, DType out_dt);

// The same for experts with a gate: per expert [gate (ff) | up (ff)] in z's columns;
// act(gate) * up * weights[row, expert] as [n, n_experts ff] in out_dt.
Buf gated_weighted(Device &d, const Stack &z, const float *weights, int w_ld, int n_experts, long long ff,
                   int kind, DType out_dt);

// A causal convolution over time on C columns (from col0) of a product's sums u, without
// the input added: act(bias + sum_j w[:, j] u_{t - taps + 1 + j}) as [n, C] in out_dt (act:
// "" or "silu"; bias float32 [C] or null; w float32 [C, taps]).  state: float32
// [taps - 1, C] per slot, slot_stride floats apart.  write_out / write_state as short_conv.
Buf causal_conv(Device &d, const Stack &u, long long col0, long long C, const float *w, const float *bias,
                int taps, float *state, long long slot_stride, const int32_t *row_pos, const int32_t *row_seq,
                const int32_t *seq_slot, bool silu, DType out_dt, bool write_out, bool write_state);

// A recurrence with a matrix of N x P values per head as state (csrc/matrix_state.cu):
// S_t = a_t S_{t-1} + b_t k_t v_t^T, y_t = S_t^T q_t + d v_t; y comes back as float32 [n, H P].
// src holds v (H P columns from val_col0), k and q (G N columns each).  With dt (the steps'
// sums, H columns from dt_col0): a = exp(-exp(a_log) softplus(dt + dt_bias)), b = that
// softplus, d = skip; without: a = decay[h], b = 1, d = 0.  silu: v, k, q are silu(sum).
// state: float32 [H, N, P] per slot, slot_stride floats apart.
struct MatrixScan {
    int H = 0, G = 0, N = 0, P = 0;
    long long val_col0 = 0, key_col0 = 0, qry_col0 = 0, dt_col0 = 0;
    bool silu = false;
    const Stack *dt = nullptr;
    const float *dt_bias = nullptr, *a_log = nullptr, *skip = nullptr, *decay = nullptr;
};
// max_len: the most rows that one sequence brings (0: not known); long sequences are then cut
// into pieces that run side by side, with a pass between them that carries the state along.
Buf matrix_state_scan(Device &d, const Stack &src, const MatrixScan &m, float *state, long long slot_stride,
                      const int32_t *row_seq, const int32_t *seq_slot, int n_seqs, bool every_row_starts,
                      long long max_len = 0);
// rms(y * silu(pre)) in `parts` equal parts of the row, times w, times sigmoid(post): y float32
// [n, width]; pre / post: sums whose columns from pre_col0 / post_col0 are read (null: none).
// few_rows: the bfloat16 path's kernel for a decode step's rows (a cluster of CTAs per row and part).
Buf gated_part_norm(Device &d, const float *y, long long n, long long width, int parts, const Stack *pre,
                    long long pre_col0, const Stack *post, long long post_col0, const float *w, float eps,
                    DType out_dt, bool few_rows = false);
// Two results as one stack of one sum: sl * sum(L) + sr * sum(R), or with weights (float32
// [m] each) sl * rms(sum L) wl + sr * rms(sum R) wr.
// few_rows: the bfloat16 path's kernel for a decode step's rows (a cluster of CTAs per row).
Stack pair_combine(Device &d, const Stack &L, const Stack &R, const float *wl, const float *wr, float sl,
                   float sr, float eps, bool few_rows = false);
// gelu_tanh(sum P) * table[tokens[row], col0 .. col0 + dim - 1] as [n, dim] in out_dt
Buf token_gate(Device &d, const Stack &P, const DevTensor &table, long long col0, long long dim,
               const int32_t *tokens, DType out_dt);

// RMSNorm of the rows of x (float32 [n, dm]).  With delta, x is first updated in
// place, x += delta[0] + ... + delta[S-1].  With rows (n_out int32 indices on the
// device) only those rows are normalized and returned, in that order; delta and
// rows together: the add runs first, as a launch of its own.
Buf rmsnorm(Device &d, float *x, long long n, long long dm, const DevTensor &weight, float eps,
            DType out_dt, const Stack *delta, const int32_t *rows, long long n_out);
void add_(Device &d, float *x, long long n, long long dm, const Stack &delta);
// y[r, :] += bias for every row of y (float32 [n, m])
void add_bias_(Device &d, float *y, long long n, long long m, const float *bias);

// SiLU(gate) * up for a stack [S, n, 2 ff] whose columns are [gate | up]
Buf swiglu(Device &d, const Stack &gate_up, DType out_dt);

// cos and sin of (float)p * inv_freq[i] for p < n_pos: two float32 [n_pos, half]
void rope_table(Device &d, const float *inv_freq_dev, int half, long long n_pos, float *cos_out,
                float *sin_out);

// a [n, k] . weight[m, k]^T as a stack of float32 partial sums.  bfloat16 operands
// whose rows are a multiple of 8 long go to the tensor-core kernel (which may cut
// k into S parts); everything else goes to the plain multiply-add kernel, S = 1.
// whole: S = 1 in every case.
Stack linear(Device &d, const void *a, DType a_dt, long long n, long long k, const DevTensor &weight,
             bool whole = false, bool force_simt = false, int splits = 0);
// One product per head: a [H, n, k] (one head's rows together) . w[H m, k]^T, head h
// with rows h m .. h m + m - 1 of w.  The result: float32 [H, S, n, m].
struct HeadStack {
    Buf buf;
    int H = 0, S = 0;
    long long n = 0, m = 0;
    float *data() const { return (float *)buf.ptr; }
};
HeadStack linear_heads(Device &d, const void *a, DType a_dt, int H, long long n, long long k,
                       const DevTensor &w);
// Into how many parts of k the tensor-core product is cut when the caller leaves it open.
int linear_parts(long long n, long long m, long long k);
// SiLU(a . gate^T) * (a . up^T) in one tensor-core kernel; an empty Buf when the
// kernel does not take the operands.  Output bfloat16 [n, ff].
Buf linear_swiglu(Device &d, const void *a, DType a_dt, long long n, long long k,
                  const DevTensor &gate_up);

struct AttnGeometry {
    int nh = 0, nkv = 0, hd = 0, window = 0;
    float scale = 1.0f;
    float softcap = 0.0f;                    // > 0: a score s becomes softcap * tanh(s / softcap)
    const float *slopes = nullptr;           // float32 [nh]: slope * (distance back) is taken off a score
    int vd = 0;                              // the values' head size; 0: as the keys'
    const float *head_scale = nullptr;       // float32 [nh] on the device: a factor per head on the scores
    const float *sink = nullptr;             // float32 [nh]: exp(sink) joins each softmax's denominator
    bool head_scale_positive = true;         // every factor is > 0 (the prefill tensor-core kernel needs it)
    int keep_first = 0;                      // with a window: the first positions stay visible to all later rows
    const float *score_bias = nullptr;       // float32 [nh]: a key's weight is sigmoid(score + bias), not normalized
    int value_dim() const { return vd > 0 ? vd : hd; }
};

// what the attention kernels see of the cache and of the step's index arrays
struct AttnCache {
    void *k = nullptr, *v = nullptr;       // [pages, kv_heads, PAGE, head_dim]
    long long n_pages = 0;
    DType dt = F32;
    const int32_t *block_table = nullptr;  // [sequences, bt_stride]
    int bt_stride = 0;
    bool writes = true;
    int v_ld = 0;                          // the length of v's rows where it is not the values' head size
};

// Per-head RMSNorm of q and k (when weights are given), NeoX rotation by the rows'
// positions (when tables are given), K and V appended to the cache pages (when the
// cache writes).  qkv: stack [S, n, (heads + 2 kv_heads) head_dim].  Returns q
// [n, heads, head_dim] in out_dt.
Buf qk_norm_rope_append(Device &d, const Stack &qkv, const DevTensor *q_w, const DevTensor *k_w,
                        float eps, const float *cos, const float *sin, const int32_t *row_pos,
                        const int32_t *row_seq, const AttnCache &c, const AttnGeometry &g,
                        DType out_dt);

// The fused [q | k | v] product's sums plus a bias (float32 over the product's
// columns, or null): q [n, heads, hd] in out_dt comes back, K and V go to the
// cache pages at the rows' positions.  With append false the product holds q alone
// (a mixer that reads another's keys and values).
Buf qkv_bias_append(Device &d, const Stack &qkv, const float *bias, const int32_t *row_pos,
                    const int32_t *row_seq, const AttnCache &c, const AttnGeometry &g, DType out_dt,
                    bool append, float q_coef = 0.0f, int q_every = 0);

// The element-wise steps of latent attention (csrc/latent.cu).  P: the down products'
// sums; the RMS-normed query latent [n, q_rank] comes back in out_dt, the row
// [RMS-normed latent | rotated shared key part] goes to the cache at each row's position.
Buf latent_down(Device &d, const Stack &P, long long q_col0, long long q_rank, const float *wq,
                long long kv_col0, long long kv_rank, const float *wkv, long long rot_dim,
                const float *cos, const float *sin, int rot_half, const int32_t *row_pos,
                const int32_t *row_seq, const AttnCache &c, float eps, DType out_dt, Buf *rows_out = nullptr);
// Q: the query product's sums [S, n, nh (D + R)] -> the plain parts [nh, n, D] (returned)
// and the rotated parts in columns C.. of q_lat [n, nh, C + R]
Buf latent_q_split(Device &d, const Stack &Q, int nh, long long D, long long R, long long C,
                   const float *cos, const float *sin, int rot_half, const int32_t *row_pos,
                   void *q_lat, DType dt, bool plain_head_major = true);
// A product that holds keys and values alone, [k | v] per row: into the cache pages at
// the rows' positions (c.k, c.v, c.block_table; kv_heads heads of hd and vd values).
void kv_append(Device &d, const Stack &kv, const int32_t *row_pos, const int32_t *row_seq,
               const AttnCache &c, int kv_heads, int hd, int vd);
// a [n, width] in dt, times sigmoid of the gate's sums (columns g_col0.. of g): [n, width] in dt
Buf gate_rows(Device &d, const void *a, DType dt, long long n, long long width, const Stack &g,
              long long g_col0);
void latent_q_join(Device &d, const HeadStack &A, long long R, void *q_lat, DType dt);
// per-head sums joined into rows [n, H m], times sigmoid of the gate's sums (columns
// g_col0.. of g; an empty g: no gate)
Buf heads_gate(Device &d, const HeadStack &A, const Stack &g, long long g_col0, DType out_dt);
// w viewed as [H, rows / H, cols] -> [H, cols, rows / H], a new tensor of the same type
DevTensor transpose_heads(Device &d, const DevTensor &w, int H);

// q, k, v out of the fused product's sums (bias: float32 over its columns or null): per-head
// RMS norm of q and k (weights float32 [hd], or null), rotation of the first 2 rot_half
// values of a head, K and V (of their own head size) into the cache.  Returns q [n, heads, hd].
// pairs: the rotation turns neighbours (2i, 2i + 1) by angle i instead of (i, i + rot_half);
// unit_norm: q and k heads are divided by their root mean square (eps inside the root)
// after the rotation, without a weight.
Buf qkv_prepare_append(Device &d, const Stack &qkv, const float *bias, const float *q_w, const float *k_w,
                       float eps, const float *cos, const float *sin, int rot_half, const int32_t *row_pos,
                       const int32_t *row_seq, const AttnCache &c, const AttnGeometry &g, DType out_dt,
                       bool pairs = false, bool unit_norm = false);
// chunks that the kept first tokens of a windowed mixer add to a row's range
int attention_kept_chunks(int window, int keep_first);

// The blocks a prefill step is cut into for the tensor-core kernel: int32
// [blocks, 4] = first row, positions, the first row's position, sequence;
// uploaded to a temporary.  n_blocks comes back.
Buf attention_blocks(Device &d, const long long *seq_row0, const long long *seq_pos0,
                     const long long *seq_len, int n_seqs, int positions_per_block, int *n_blocks);
int attention_block_positions(int nh, int nkv);
bool attention_tc_ok(int nh, int nkv, int hd);

// Causal GQA attention of every row over its sequence's cache pages: q [n, heads,
// hd] of the cache's dtype -> out of the same shape and dtype.  max_chunks: the
// most chunks of attention_chunk() positions that any row's range touches.
// bfloat16 heads of 64 or 128 values run on the tensor cores when the caller says
// how the rows are arranged: decode (every row is the one new token of its
// sequence) or blocks (from attention_blocks).
Buf attention(Device &d, const void *q, long long n, const AttnCache &c, const AttnGeometry &g,
              const int32_t *row_pos, const int32_t *row_seq, int max_chunks, const int32_t *blocks,
              int n_blocks, bool decode, bool force_simt = false, bool head_major = false);

// qk_norm_rope_append and attention(decode) in one kernel, from the q,k,v product's
// partial sums; an empty Buf where the kernel does not take these sizes and types.
// bias: float32 over the product's columns, added to its sums, or null.
Buf attention_decode_qkv(Device &d, const Stack &qkv, const DevTensor *q_w, const DevTensor *k_w,
                         float eps, const float *cos, const float *sin, const AttnCache &c,
                         const AttnGeometry &g, const int32_t *row_pos, const int32_t *row_seq,
                         int max_chunks, const float *bias = nullptr);

struct SamplerArrays {
    const int32_t *row_slot = nullptr;
    const float *temperature = nullptr;   // null: every row takes its first maximum
    const int32_t *top_k = nullptr;
    const float *top_p = nullptr, *min_p = nullptr;
    unsigned long long *rng = nullptr;
    unsigned long long *big_keys = nullptr;   // [rows, big_cap] or null
    float *big_probs = nullptr;
    long long big_cap = 0;
    int32_t *forced = nullptr;
};
// One token per row of logits [rows, V] into out (int32 [rows] on the device).
void sample(Device &d, const float *logits, int rows, int vocab, const SamplerArrays &s, int32_t *out);

// 0, or which bounded wait of a tensor-core kernel ran out since the last call
// (the kernels' output is then not valid).  Both synchronize the device.
int gemm_tc_error();
int attn_tc_error();

}  // namespace ops
}  // namespace jb

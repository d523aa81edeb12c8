#include "launch.h"

#include <algorithm>
#include <atomic>
#include <vector>

#include "../cache/cache.h"
#include "kernels.h"

namespace jb {
namespace ops {

static std::atomic<long long> g_launches{0};

long long launches() { return g_launches.load(); }
void count_launches(long long n) { g_launches += n; }

static void check(int code, const char *what, int kernels = 1) {
    if (code == 0) {
        g_launches += kernels;
        return;
    }
    if (code == -1) fail(JB_LLM_EINVAL, std::string(what) + ": the kernel does not take these sizes or types");
    cudaError_t e = cudaGetLastError();
    fail(JB_LLM_EFAIL, fmt("%s: the launch failed (code %d%s%s)", what, code, e != cudaSuccess ? ": " : "",
                           e != cudaSuccess ? cudaGetErrorString(e) : ""));
}

static void need_float(DType dt, const char *what) {
    if (dt != F32 && dt != BF16) fail(JB_LLM_EINVAL, std::string(what) + ": float32 or bfloat16 is needed");
}

static int as_int(long long v, const char *what) {
    if (v < 0 || v > 0x7fffffffll) fail(JB_LLM_EINVAL, std::string(what) + ": too large for the kernels");
    return (int)v;
}

int attention_chunk() { return jb_attention_chunk(); }
int sample_small_cap() { return jb_sample_small_cap(); }
bool sample_needs_big(int vocab, int top_k) { return jb_sample_needs_big(vocab, top_k) != 0; }

// ------------------------------------------------------------------ row-wise
Buf embed(Device &d, const DevTensor &table, const int32_t *tokens, long long n, const DevTensor *pos_table,
          const int32_t *row_pos) {
    need_float(table.dt, "embedding table");
    long long dm = table.shape.at(1);
    Buf x = d.pool.get((size_t)n * (size_t)dm * 4);
    if (pos_table) {
        need_float(pos_table->dt, "position table");
        if (pos_table->shape.size() != 2 || pos_table->shape[1] != dm || !row_pos)
            fail(JB_LLM_EINVAL, "embed: the position table's rows are not as wide as the embedding's");
        check(jb_embed_pos(table.ptr, table.dt, pos_table->ptr, pos_table->dt, tokens, row_pos, x.as<float>(),
                           as_int(n, "rows"), as_int(dm, "width"), d.stream), "embed");
        return x;
    }
    check(jb_embed(table.ptr, table.dt, tokens, x.as<float>(), as_int(n, "rows"), as_int(dm, "width"),
                   d.stream), "embed");
    return x;
}

Buf dyt(Device &d, float *x, long long n, long long dm, const DytParams &p, DType out_dt, const Stack *delta,
        const int32_t *rows, long long n_out) {
    need_float(out_dt, "norm output");
    if (delta && rows) {
        add_(d, x, n, dm, *delta);
        delta = nullptr;
    }
    if (delta && (delta->n != n || delta->m != dm)) fail(JB_LLM_EINVAL, "dyt: delta's shape is not x's");
    if (delta) resolve_bias(d, const_cast<Stack &>(*delta));
    long long outs = rows ? n_out : n;
    Buf out = d.pool.get((size_t)outs * (size_t)dm * dtype_size(out_dt));
    check(jb_dyt(x, delta ? delta->data() : nullptr, delta ? delta->S : 0, delta ? delta->stride() : 0, rows,
                 p.w, p.b, p.alpha, out.ptr, out_dt, as_int(outs, "rows"), as_int(dm, "width"), d.stream),
          "dyt");
    return out;
}

static void gate_shapes(const Stack &y, const Stack &g, long long g_col0, const char *what) {
    if (g.n != y.n || g_col0 < 0 || g_col0 + y.m > g.m)
        fail(JB_LLM_EINVAL, std::string(what) + ": the gate does not cover the sublayer's result");
}

Buf gate_mul(Device &d, const Stack &y, const Stack &g, long long g_col0, const float *g_bias) {
    const float *y_bias = y.bias;
    gate_shapes(y, g, g_col0, "gate_mul");
    Buf out = d.pool.get((size_t)y.n * (size_t)y.m * 4);
    check(jb_gate_mul(y.data(), y.S, y.stride(), y_bias, g.data(), g.S, g.stride(), as_int(g.m, "width"),
                      (int)g_col0, g_bias, out.as<float>(), as_int(y.n, "rows"), as_int(y.m, "width"),
                      d.stream), "gate_mul");
    return out;
}

Buf gated_dyt_residual(Device &d, float *x, const Stack &y, const Stack &g, long long g_col0,
                       const float *g_bias, const DytParams &post, const DytParams *next, DType out_dt) {
    const float *y_bias = y.bias;
    gate_shapes(y, g, g_col0, "gated_dyt_residual");
    Buf out;
    if (next) {
        need_float(out_dt, "norm output");
        out = d.pool.get((size_t)y.n * (size_t)y.m * dtype_size(out_dt));
    }
    check(jb_gated_dyt_residual(x, y.data(), y.S, y.stride(), y_bias, g.data(), g.S, g.stride(),
                                as_int(g.m, "width"), (int)g_col0, g_bias, post.w, post.b, post.alpha,
                                next ? next->w : nullptr, next ? next->b : nullptr,
                                next ? next->alpha : nullptr, out.ptr, out_dt, as_int(y.n, "rows"),
                                as_int(y.m, "width"), out_dt == BF16 ? 1 : 0, d.stream), "gated_dyt_residual");
    return out;
}

Buf polynorm(Device &d, const Stack &z, long long ff, const float *coef, float eps, DType out_dt) {
    need_float(out_dt, "activation output");
    if (ff <= 0 || ff > z.m) fail(JB_LLM_EINVAL, "polynorm: the product is narrower than the feed-forward");
    Buf out = d.pool.get((size_t)z.n * (size_t)ff * dtype_size(out_dt));
    check(jb_polynorm(z.data(), z.S, z.stride(), as_int(z.m, "width"), coef, eps, out.ptr, out_dt,
                      as_int(z.n, "rows"), as_int(ff, "width"), d.stream), "polynorm");
    return out;
}

void scale_(Device &d, float *x, long long total, float s) {
    check(jb_scale(x, s, total, d.stream), "scale");
}

Buf qkv_bias_append(Device &d, const Stack &qkv, const float *bias, const int32_t *row_pos,
                    const int32_t *row_seq, const AttnCache &c, const AttnGeometry &g, DType out_dt,
                    bool append, float q_coef, int q_every) {
    long long width = (long long)g.nh * g.hd + (append ? (long long)g.nkv * (g.hd + g.value_dim()) : 0);
    if (qkv.m < width) fail(JB_LLM_EINVAL, "qkv_bias_append: the product is narrower than q, k and v");
    if (append && (!c.k || !c.v)) fail(JB_LLM_EINVAL, "qkv_bias_append: no cache to append to");
    if (append && c.dt != out_dt) fail(JB_LLM_EINVAL, "qkv_bias_append: the cache is of another type");
    Buf q = d.pool.get((size_t)qkv.n * (size_t)g.nh * (size_t)g.hd * dtype_size(out_dt));
    if (q_every < 0) fail(JB_LLM_EINVAL, "qkv_bias_append: the query temperature's step must not be negative");
    check(jb_qkv_bias_append_temp(qkv.data(), qkv.S, qkv.stride(), as_int(qkv.m, "width"), bias, row_pos,
                                  row_seq, c.block_table, c.bt_stride, q.ptr, append ? c.k : nullptr,
                                  append ? c.v : nullptr, out_dt, as_int(qkv.n, "rows"), g.nh, g.nkv, g.hd,
                                  g.value_dim(), append ? 1 : 0, q_coef, q_every, d.stream),
          "qkv_bias_append");
    return q;
}

Buf layernorm(Device &d, float *x, long long n, long long dm, const LnParams &p, DType out_dt,
              const Stack *a, const Stack *b, float mult, const int32_t *rows, long long n_out) {
    need_float(out_dt, "norm output");
    if (!a && b) { a = b; b = nullptr; }
    if (a && rows) {
        add_scaled_(d, x, n, dm, *a, b, mult);
        a = b = nullptr;
    }
    for (const Stack *s : {a, b}) {
        if (!s) continue;
        if (s->n != n || s->m != dm) fail(JB_LLM_EINVAL, "layernorm: a sum's shape is not x's");
        resolve_bias(d, const_cast<Stack &>(*s));
    }
    long long outs = rows ? n_out : n;
    Buf out = d.pool.get((size_t)outs * (size_t)dm * dtype_size(out_dt));
    check(jb_layernorm(x, a ? a->data() : nullptr, a ? a->S : 0, a ? a->stride() : 0, b ? b->data() : nullptr,
                       b ? b->S : 0, b ? b->stride() : 0, mult, rows, p.w, p.b, out.ptr, out_dt,
                       as_int(outs, "rows"), as_int(dm, "width"), p.eps, d.stream), "layernorm");
    return out;
}

void add_scaled_(Device &d, float *x, long long n, long long dm, const Stack &a, const Stack *b, float mult) {
    for (const Stack *s : {&a, b}) {
        if (!s) continue;
        if (s->n != n || s->m != dm) fail(JB_LLM_EINVAL, "add_scaled: a sum's shape is not x's");
        resolve_bias(d, const_cast<Stack &>(*s));
    }
    check(jb_layernorm(x, a.data(), a.S, a.stride(), b ? b->data() : nullptr, b ? b->S : 0,
                       b ? b->stride() : 0, mult, nullptr, nullptr, nullptr, nullptr, 0, as_int(n, "rows"),
                       as_int(dm, "width"), 0.0f, d.stream), "add_scaled");
}

void norm_residual_(Device &d, float *x, const Stack &y, const LnParams &p, bool rms, bool few_rows) {
    if (!y) fail(JB_LLM_EINVAL, "norm_residual: no result to norm");
    check(jb_norm_residual(x, y.data(), y.S, y.stride(), y.bias, y.skip, y.skip_dt, y.skip_coef,
                           (int)y.skip_coef_ld, p.w, p.b, as_int(y.n, "rows"), as_int(y.m, "width"), p.eps,
                           rms ? 1 : 0, few_rows ? 1 : 0, d.stream), "norm_residual");
}

Buf short_conv(Device &d, const float *x, long long n, long long dm, const float *w, int taps, float *state,
               long long slot_stride, const int32_t *row_pos, const int32_t *row_seq, const int32_t *seq_slot, DType out_dt,
               bool write_h, bool write_state) {
    need_float(out_dt, "short_conv output");
    Buf out;
    if (write_h) out = d.pool.get((size_t)n * (size_t)dm * dtype_size(out_dt));
    int what = (write_h ? 1 : 0) | (write_state ? 2 : 0);
    if (!what) return out;
    check(jb_short_conv(x, w, state, slot_stride, row_pos, row_seq, seq_slot, out.ptr, out_dt, as_int(n, "rows"),
                        as_int(dm, "width"), taps, what, d.stream), "short_conv");
    return out;
}

Buf mingru(Device &d, const Stack &P, long long col0, long long W, const float *bias, float *state,
           const int32_t *row_seq, const int32_t *seq_slot, int n_seqs, bool every_row_starts, DType out_dt) {
    need_float(out_dt, "mingru output");
    if (P.m < col0 + 3 * W) fail(JB_LLM_EINVAL, "mingru: the product is narrower than z, x and g");
    int n = as_int(P.n, "rows"), w = as_int(W, "width");
    long long need = jb_mingru_scratch(n, n_seqs, w, every_row_starts ? 1 : 0);
    Buf scratch;
    if (need > 0) scratch = d.pool.get((size_t)need * 4);
    Buf out = d.pool.get((size_t)P.n * (size_t)W * dtype_size(out_dt));
    check(jb_mingru(P.data(), P.S, P.stride(), as_int(P.m, "width"), (int)col0, bias, state, row_seq, seq_slot,
                    scratch.as<float>(), out.ptr, out_dt, n, n_seqs, w, every_row_starts ? 1 : 0, d.stream),
          "mingru", need > 0 ? 3 : 1);
    return out;
}

Buf moe_route(Device &d, const Stack &P, long long col0, const RouteParams &r, Buf *skip_coef) {
    if (P.m < col0 + r.experts) fail(JB_LLM_EINVAL, "moe_route: the product is narrower than the router's rows");
    Buf weights = d.pool.get(std::max<size_t>((size_t)P.n * (size_t)r.experts * 4, 16));
    if (skip_coef) *skip_coef = d.pool.get(std::max<size_t>((size_t)P.n * 4, 16));
    check(jb_moe_route(P.data(), P.S, P.stride(), as_int(P.m, "width"), (int)col0, r.correction,
                       weights.as<float>(), skip_coef ? skip_coef->as<float>() : nullptr, as_int(P.n, "rows"),
                       r.experts, r.groups, r.keep, r.top, r.first_identity, r.scale, r.sigmoid_scores ? 1 : 0,
                       r.group_best, d.stream), "moe_route");
    return weights;
}

Buf gated_weighted(Device &d, const Stack &z, const float *weights, int w_ld, int n_experts, long long ff,
                   int kind, DType out_dt) {
    need_float(out_dt, "activation output");
    long long width = (long long)n_experts * ff;
    if (width <= 0 || 2 * width > z.m) fail(JB_LLM_EINVAL, "gated_weighted: the product is narrower than the experts");
    Buf out = d.pool.get((size_t)z.n * (size_t)width * dtype_size(out_dt));
    check(jb_gated_weighted(z.data(), z.S, z.stride(), as_int(z.m, "width"), weights, w_ld, n_experts,
                            as_int(ff, "width"), kind, out.ptr, out_dt, as_int(z.n, "rows"), d.stream),
          "gated_weighted");
    return out;
}

Buf causal_conv(Device &d, const Stack &u, long long col0, long long C, const float *w, const float *bias,
                int taps, float *state, long long slot_stride, const int32_t *row_pos, const int32_t *row_seq,
                const int32_t *seq_slot, bool silu, DType out_dt, bool write_out, bool write_state) {
    need_float(out_dt, "causal_conv output");
    if (!u || col0 < 0 || C <= 0 || col0 + C > u.m) fail(JB_LLM_EINVAL, "causal_conv: the columns lie outside the product");
    Buf out;
    if (write_out) out = d.pool.get((size_t)u.n * (size_t)C * dtype_size(out_dt));
    int what = (write_out ? 1 : 0) | (write_state && taps > 1 ? 2 : 0);
    if (!what) return out;
    check(jb_causal_conv(u.data(), u.S, u.stride(), as_int(u.m, "width"), (int)col0, w, bias, state, slot_stride,
                         row_pos, row_seq, seq_slot, out.ptr, out_dt, as_int(C, "width"), as_int(u.n, "rows"),
                         as_int(C, "width"), taps, silu ? 1 : 0, what, d.stream), "causal_conv");
    return out;
}

Buf matrix_state_scan(Device &d, const Stack &src, const MatrixScan &m, float *state, long long slot_stride,
                      const int32_t *row_seq, const int32_t *seq_slot, int n_seqs, bool every_row_starts,
                      long long max_len) {
    if (!src || !state) fail(JB_LLM_EINVAL, "matrix_state_scan: no input or no state");
    if (m.dt && m.dt->n != src.n) fail(JB_LLM_EINVAL, "matrix_state_scan: the steps are of other rows");
    Buf y = d.pool.get(std::max<size_t>((size_t)src.n * (size_t)m.H * (size_t)m.P * 4, 16));
    long long need = every_row_starts ? 0 : jb_matrix_state_scratch(n_seqs, (int)std::min<long long>(max_len, 0x7fffffff),
                                                                     m.H, m.N, m.P);
    Buf scratch;
    if (need > 0) scratch = d.pool.get((size_t)need * 4);
    check(jb_matrix_state_scan(src.data(), src.S, src.stride(), as_int(src.m, "width"), (int)m.val_col0,
                               (int)m.key_col0, (int)m.qry_col0, m.silu ? 1 : 0, m.dt ? m.dt->data() : nullptr,
                               m.dt ? m.dt->S : 0, m.dt ? m.dt->stride() : 0, m.dt ? as_int(m.dt->m, "width") : 0,
                               (int)m.dt_col0, m.dt_bias, m.a_log, m.skip, m.decay, state, slot_stride, row_seq,
                               seq_slot, y.as<float>(), as_int(src.n, "rows"), n_seqs, m.H, m.G, m.N, m.P,
                               every_row_starts ? 1 : 0, need > 0 ? scratch.as<float>() : nullptr,
                               (int)std::min<long long>(max_len, 0x7fffffff), d.stream),
          "matrix_state_scan", need > 0 ? 3 : 1);
    return y;
}

Buf gated_part_norm(Device &d, const float *y, long long n, long long width, int parts, const Stack *pre,
                    long long pre_col0, const Stack *post, long long post_col0, const float *w, float eps,
                    DType out_dt, bool few_rows) {
    need_float(out_dt, "gated_part_norm output");
    if ((pre && pre->n != n) || (post && post->n != n)) fail(JB_LLM_EINVAL, "gated_part_norm: a gate of other rows");
    Buf out = d.pool.get(std::max<size_t>((size_t)n * (size_t)width * dtype_size(out_dt), 16));
    check(jb_gated_part_norm(y, pre ? pre->data() : nullptr, pre ? pre->S : 0, pre ? pre->stride() : 0,
                             pre ? as_int(pre->m, "width") : 0, (int)pre_col0, post ? post->data() : nullptr,
                             post ? post->S : 0, post ? post->stride() : 0, post ? as_int(post->m, "width") : 0,
                             (int)post_col0, w, eps, out.ptr, out_dt, as_int(n, "rows"), as_int(width, "width"),
                             parts, few_rows ? 1 : 0, d.stream), "gated_part_norm");
    return out;
}

Stack pair_combine(Device &d, const Stack &L, const Stack &R, const float *wl, const float *wr, float sl,
                   float sr, float eps, bool few_rows) {
    if (!L || !R || L.n != R.n || L.m != R.m) fail(JB_LLM_EINVAL, "pair_combine: the two results differ in shape");
    if (L.bias || R.bias || L.skip || R.skip) fail(JB_LLM_EINVAL, "pair_combine: a result still has a term to be added");
    Stack out;
    out.S = 1;
    out.n = L.n;
    out.m = L.m;
    out.buf = d.pool.get(std::max<size_t>((size_t)L.n * (size_t)L.m * 4, 16));
    check(jb_pair_combine(L.data(), L.S, L.stride(), R.data(), R.S, R.stride(), wl, wr, sl, sr, eps, out.data(),
                          as_int(L.n, "rows"), as_int(L.m, "width"), few_rows ? 1 : 0, d.stream), "pair_combine");
    return out;
}

Buf token_gate(Device &d, const Stack &P, const DevTensor &table, long long col0, long long dim,
               const int32_t *tokens, DType out_dt) {
    need_float(out_dt, "token_gate output");
    if (!P || P.m < dim || table.shape.size() != 2 || col0 < 0 || col0 + dim > table.shape[1])
        fail(JB_LLM_EINVAL, "token_gate: the columns lie outside the table or the product");
    Buf out = d.pool.get(std::max<size_t>((size_t)P.n * (size_t)dim * dtype_size(out_dt), 16));
    check(jb_token_gate(P.data(), P.S, P.stride(), as_int(P.m, "width"), table.ptr, table.dt,
                        as_int(table.shape[1], "width"), (int)col0, tokens, out.ptr, out_dt, as_int(P.n, "rows"),
                        as_int(dim, "width"), d.stream), "token_gate");
    return out;
}

Buf activation_weighted(Device &d, const Stack &z, long long width, const float *weights, int w_ld, int n_experts,
                        long long ff, int kind, DType out_dt) {
    need_float(out_dt, "activation output");
    if (width <= 0 || width > z.m) fail(JB_LLM_EINVAL, "activation_weighted: the product is narrower than the experts");
    Buf out = d.pool.get((size_t)z.n * (size_t)width * dtype_size(out_dt));
    check(jb_activation_weighted(z.data(), z.S, z.stride(), as_int(z.m, "width"), weights, w_ld, n_experts,
                                 as_int(ff, "width"), kind, out.ptr, out_dt, as_int(z.n, "rows"),
                                 as_int(width, "width"), d.stream), "activation_weighted");
    return out;
}

Buf qkv_prepare_append(Device &d, const Stack &qkv, const float *bias, const float *q_w, const float *k_w,
                       float eps, const float *cos, const float *sin, int rot_half, const int32_t *row_pos,
                       const int32_t *row_seq, const AttnCache &c, const AttnGeometry &g, DType out_dt,
                       bool pairs, bool unit_norm) {
    bool append = c.writes;
    long long width = (long long)g.nh * g.hd + (append ? (long long)g.nkv * (g.hd + g.value_dim()) : 0);
    if (qkv.m < width) fail(JB_LLM_EINVAL, "qkv_prepare_append: the product is narrower than q, k and v");
    if (append && (!c.k || !c.v)) fail(JB_LLM_EINVAL, "qkv_prepare_append: no cache to append to");
    if (append && c.dt != out_dt) fail(JB_LLM_EINVAL, "qkv_prepare_append: the cache is of another type");
    Buf q = d.pool.get((size_t)qkv.n * (size_t)g.nh * (size_t)g.hd * dtype_size(out_dt));
    check(jb_qkv_prepare_append(qkv.data(), qkv.S, qkv.stride(), as_int(qkv.m, "width"), bias, q_w, k_w, eps, cos,
                                sin, rot_half, row_pos, row_seq, c.block_table, c.bt_stride, q.ptr,
                                append ? c.k : nullptr, append ? c.v : nullptr, out_dt, as_int(qkv.n, "rows"),
                                g.nh, g.nkv, g.hd, g.value_dim(),
                                (pairs ? JB_ROT_PAIRS : 0) | (unit_norm ? JB_UNIT_NORM : 0), d.stream),
          "qkv_prepare_append");
    return q;
}

int attention_kept_chunks(int window, int keep_first) { return jb_attention_kept_chunks(window, keep_first); }

int activation_kind(const std::string &name) {
    if (name == "relu2") return JB_ACT_RELU2;
    if (name == "relu") return JB_ACT_RELU;
    if (name == "gelu_tanh") return JB_ACT_GELU_TANH;
    if (name == "silu") return JB_ACT_SILU;
    return -1;
}

Buf activation(Device &d, const Stack &z, long long ff, int kind, DType out_dt, long long col0) {
    need_float(out_dt, "activation output");
    if (ff <= 0 || col0 < 0 || col0 + ff > z.m) fail(JB_LLM_EINVAL, "activation: the product is narrower than the feed-forward");
    Buf out = d.pool.get((size_t)z.n * (size_t)ff * dtype_size(out_dt));
    check(jb_activation(z.data() + col0, z.S, z.stride(), as_int(z.m, "width"), kind, out.ptr, out_dt,
                        as_int(z.n, "rows"), as_int(ff, "width"), d.stream), "activation");
    return out;
}

// ------------------------------------------------------------ latent attention
Buf latent_down(Device &d, const Stack &P, long long q_col0, long long q_rank, const float *wq,
                long long kv_col0, long long kv_rank, const float *wkv, long long rot_dim, const float *cs,
                const float *sn, int rot_half, const int32_t *row_pos, const int32_t *row_seq,
                const AttnCache &c, float eps, DType out_dt, Buf *rows_out) {
    if (!c.k || !c.writes) fail(JB_LLM_EINVAL, "latent_down: no cache to write the latent to");
    if (c.dt != out_dt) fail(JB_LLM_EINVAL, "latent_down: the cache is of another type");
    Buf cq = d.pool.get(std::max<size_t>((size_t)P.n * (size_t)q_rank * dtype_size(out_dt), 16));
    if (rows_out) *rows_out = d.pool.get((size_t)P.n * (size_t)(kv_rank + rot_dim) * dtype_size(out_dt));
    check(jb_latent_down_rows(P.data(), P.S, P.stride(), as_int(P.m, "width"), (int)q_col0, (int)q_rank, wq,
                              (int)kv_col0, (int)kv_rank, wkv, (int)rot_dim, cs, sn, rot_half, row_pos,
                              row_seq, c.block_table, c.bt_stride, cq.ptr, c.k,
                              rows_out ? rows_out->ptr : nullptr, out_dt, as_int(P.n, "rows"), eps,
                              d.stream), "latent_down");
    return cq;
}

Buf latent_q_split(Device &d, const Stack &Q, int nh, long long D, long long R, long long C, const float *cs,
                   const float *sn, int rot_half, const int32_t *row_pos, void *q_lat, DType dt,
                   bool plain_head_major) {
    if (Q.m != (long long)nh * (D + R)) fail(JB_LLM_EINVAL, "latent_q_split: the product is not heads x (plain + rotated) wide");
    if (!plain_head_major && C != D) fail(JB_LLM_EINVAL, "latent_q_split: whole queries have their plain part first");
    resolve_bias(d, const_cast<Stack &>(Q));
    Buf qp;
    if (plain_head_major) qp = d.pool.get((size_t)nh * (size_t)Q.n * (size_t)D * dtype_size(dt));
    check(jb_latent_q_split(Q.data(), Q.S, Q.stride(), nh, (int)D, (int)R, (int)C, cs, sn, rot_half, row_pos,
                            qp.ptr, q_lat, dt, as_int(Q.n, "rows"), d.stream), "latent_q_split");
    return qp;
}

void kv_append(Device &d, const Stack &kv, const int32_t *row_pos, const int32_t *row_seq, const AttnCache &c,
               int kv_heads, int hd, int vd) {
    if (kv.m < (long long)kv_heads * (hd + vd)) fail(JB_LLM_EINVAL, "kv_append: the product is narrower than k and v");
    if (!c.k || !c.v) fail(JB_LLM_EINVAL, "kv_append: no pages to append to");
    resolve_bias(d, const_cast<Stack &>(kv));
    check(jb_qkv_bias_append_temp(kv.data(), kv.S, kv.stride(), as_int(kv.m, "width"), nullptr, row_pos, row_seq,
                                  c.block_table, c.bt_stride, nullptr, c.k, c.v, c.dt, as_int(kv.n, "rows"), 0,
                                  kv_heads, hd, vd, 1, 0.0f, 0, d.stream), "kv_append");
}

Buf gate_rows(Device &d, const void *a, DType dt, long long n, long long width, const Stack &g,
              long long g_col0) {
    need_float(dt, "gate_rows");
    if (!g || g.n != n || g_col0 < 0 || g_col0 + width > g.m)
        fail(JB_LLM_EINVAL, "gate_rows: the gate does not cover the rows");
    Buf out = d.pool.get((size_t)n * (size_t)width * dtype_size(dt));
    check(jb_gate_rows(a, g.data(), g.S, g.stride(), as_int(g.m, "width"), (int)g_col0, out.ptr, dt,
                       as_int(n, "rows"), as_int(width, "width"), d.stream), "gate_rows");
    return out;
}

void latent_q_join(Device &d, const HeadStack &A, long long R, void *q_lat, DType dt) {
    check(jb_latent_q_join(A.data(), A.S, A.H, as_int(A.m, "width"), (int)R, q_lat, dt, as_int(A.n, "rows"),
                           d.stream), "latent_q_join");
}

Buf heads_gate(Device &d, const HeadStack &A, const Stack &g, long long g_col0, DType out_dt) {
    need_float(out_dt, "heads_gate output");
    if (g && (g.n != A.n || g_col0 < 0 || g_col0 + A.H * A.m > g.m))
        fail(JB_LLM_EINVAL, "heads_gate: the gate does not cover the heads' values");
    Buf out = d.pool.get((size_t)A.n * (size_t)A.H * (size_t)A.m * dtype_size(out_dt));
    check(jb_heads_gate(A.data(), A.S, A.H, as_int(A.m, "width"), g ? g.data() : nullptr, g.S, g.stride(),
                        as_int(g.m, "width"), (int)g_col0, out.ptr, out_dt, as_int(A.n, "rows"), d.stream),
          "heads_gate");
    return out;
}

DevTensor transpose_heads(Device &d, const DevTensor &w, int H) {
    need_float(w.dt, "weight");
    if (w.shape.size() != 2 || H <= 0 || w.shape[0] % H)
        fail(JB_LLM_EINVAL, "transpose_heads: the rows are not a multiple of the heads");
    long long D = w.shape[0] / H, C = w.shape[1];
    DevTensor out = d.tensor(w.dt, {(long long)H * C, D});
    check(jb_transpose_heads(w.ptr, out.ptr, w.dt, H, as_int(D, "rows"), as_int(C, "width"), d.stream),
          "transpose_heads");
    d.sync();
    return out;
}

Buf rmsnorm(Device &d, float *x, long long n, long long dm, const DevTensor &w, float eps, DType out_dt,
            const Stack *delta, const int32_t *rows, long long n_out) {
    need_float(w.dt, "norm weight");
    need_float(out_dt, "norm output");
    if (w.numel() != dm) fail(JB_LLM_EINVAL, "rmsnorm: the weight's length is not the rows' width");
    if (delta) resolve_bias(d, const_cast<Stack &>(*delta));
    if (delta && rows) {
        add_(d, x, n, dm, *delta);
        delta = nullptr;
    }
    if (delta && (delta->n != n || delta->m != dm))
        fail(JB_LLM_EINVAL, "rmsnorm: delta's shape is not x's");
    long long outs = rows ? n_out : n;
    Buf out = d.pool.get((size_t)outs * (size_t)dm * dtype_size(out_dt));
    check(jb_rmsnorm(x, delta ? delta->data() : nullptr, delta ? delta->S : 0,
                     delta ? delta->stride() : 0, rows, w.ptr, w.dt, out.ptr, out_dt, as_int(outs, "rows"),
                     as_int(dm, "width"), eps, d.stream), "rmsnorm");
    return out;
}

void add_bias_(Device &d, float *y, long long n, long long m, const float *bias) {
    check(jb_add_bias(y, bias, as_int(n, "rows"), as_int(m, "width"), d.stream), "add_bias");
}

void resolve_bias(Device &d, Stack &y) {
    if (!y) return;
    if (y.bias) {
        add_bias_(d, y.data(), y.n, y.m, y.bias);
        y.bias = nullptr;
    }
    if (y.skip) {
        check(jb_add_row_scaled(y.data(), y.skip, y.skip_dt, y.skip_coef, (int)y.skip_coef_ld, as_int(y.n, "rows"),
                                as_int(y.m, "width"), d.stream), "add_row_scaled");
        y.skip = nullptr;
        y.skip_coef = nullptr;
        y.skip_hold.reset();
    }
}

void add_(Device &d, float *x, long long n, long long dm, const Stack &delta) {
    if (delta.n != n || delta.m != dm) fail(JB_LLM_EINVAL, "add: delta's shape is not x's");
    resolve_bias(d, const_cast<Stack &>(delta));
    check(jb_rmsnorm(x, delta.data(), delta.S, delta.stride(), nullptr, nullptr, 0, nullptr, 0,
                     as_int(n, "rows"), as_int(dm, "width"), 0.0f, d.stream), "add");
}

Buf swiglu(Device &d, const Stack &gu, DType out_dt) {
    if (gu.m % 2) fail(JB_LLM_EINVAL, "swiglu: the gate_up width must be even");
    long long ff = gu.m / 2;
    Buf out = d.pool.get((size_t)gu.n * (size_t)ff * dtype_size(out_dt));
    check(jb_swiglu(gu.data(), gu.S, gu.stride(), out.ptr, out_dt, as_int(gu.n, "rows"), as_int(ff, "width"),
                    d.stream), "swiglu");
    return out;
}

void rope_table(Device &d, const float *inv, int half, long long n_pos, float *cs, float *sn) {
    check(jb_rope_table(cs, sn, inv, as_int(n_pos, "positions"), half, d.stream), "rope_table");
}

// ------------------------------------------------------------------ products
int linear_parts(long long n, long long m, long long k) {
    return jb_gemm_tc_splits((int)n, (int)m, (int)k);
}

Stack linear(Device &d, const void *a, DType a_dt, long long n, long long k, const DevTensor &w,
             bool whole, bool force_simt, int splits) {
    need_float(a_dt, "activations");
    need_float(w.dt, "weight");
    if (w.shape.size() != 2 || w.shape[1] != k)
        fail(JB_LLM_EINVAL, "linear: the weight's rows are not as long as the activations'");
    long long m = w.shape[0];
    Stack out;
    out.n = n;
    out.m = m;
    int ni = as_int(n, "rows"), mi = as_int(m, "features"), ki = as_int(k, "width");
    if (!force_simt && n > 0 && a_dt == BF16 && w.dt == BF16 && jb_gemm_tc_ok(a, w.ptr, ni, mi, ki)) {
        out.S = whole ? 1 : (splits > 0 ? splits : jb_gemm_tc_splits(ni, mi, ki));
        out.buf = d.pool.get((size_t)out.S * (size_t)n * (size_t)m * 4);
        check(jb_gemm_tc(a, w.ptr, out.data(), ni, mi, ki, out.S, d.stream), "linear (tcgen05)");
        return out;
    }
    out.S = 1;
    out.buf = d.pool.get((size_t)n * (size_t)m * 4);
    long long need = jb_gemm_simt_scratch(ni, mi, ki);
    Buf scratch;
    if (need > 0) scratch = d.pool.get((size_t)need * 4);
    check(jb_gemm_simt(a, a_dt, w.ptr, w.dt, out.data(), ni, mi, ki, scratch.as<float>(), d.stream),
          "linear", need > 0 ? 2 : 1);
    return out;
}

HeadStack linear_heads(Device &d, const void *a, DType a_dt, int H, long long n, long long k,
                       const DevTensor &w) {
    need_float(a_dt, "activations");
    need_float(w.dt, "weight");
    if (w.shape.size() != 2 || w.shape[1] != k || H <= 0 || w.shape[0] % H)
        fail(JB_LLM_EINVAL, "linear_heads: the weight is not [heads x features, width of the activations]");
    HeadStack out;
    out.H = H;
    out.n = n;
    out.m = w.shape[0] / H;
    int ni = as_int(n, "rows"), mi = as_int(out.m, "features"), ki = as_int(k, "width");
    size_t a_head = (size_t)n * (size_t)k * dtype_size(a_dt), w_head = (size_t)out.m * (size_t)k * dtype_size(w.dt);
    // the tensor-core kernel takes all heads in one launch: rows of one head follow the other's
    bool tc = n > 0 && a_dt == BF16 && w.dt == BF16 && jb_gemm_tc_ok(a, w.ptr, ni, mi, ki) != 0 &&
              (long long)H * out.m <= 0x7fffffffll && (long long)H * n <= 0x7fffffffll;
    out.S = tc ? jb_gemm_tc_splits(ni, mi, ki) : 1;
    size_t one = (size_t)out.S * (size_t)n * (size_t)out.m;
    out.buf = d.pool.get(std::max<size_t>((size_t)H * one * 4, 16));
    long long need = tc ? 0 : jb_gemm_simt_scratch(ni, mi, ki);
    Buf scratch;
    if (need > 0) scratch = d.pool.get((size_t)need * 4);
    if (tc) {
        check(jb_gemm_tc_heads(a, w.ptr, out.data(), ni, mi, ki, out.S, H, d.stream), "linear_heads (tcgen05)");
        return out;
    }
    for (int h = 0; h < H && n > 0; h++) {
        const char *ah = (const char *)a + h * a_head, *wh = (const char *)w.ptr + h * w_head;
        float *oh = out.data() + (size_t)h * one;
        check(jb_gemm_simt(ah, a_dt, wh, w.dt, oh, ni, mi, ki, scratch.as<float>(), d.stream),
              "linear_heads", need > 0 ? 2 : 1);
    }
    return out;
}

Buf linear_swiglu(Device &d, const void *a, DType a_dt, long long n, long long k, const DevTensor &gu) {
    if (gu.shape.size() != 2 || gu.shape[1] != k)
        fail(JB_LLM_EINVAL, "linear_swiglu: the weight's rows are not as long as the activations'");
    if (gu.shape[0] % 2 || n == 0 || a_dt != BF16 || gu.dt != BF16 ||
        !jb_gemm_tc_ok(a, gu.ptr, (int)n, (int)gu.shape[0], (int)k))
        return Buf();
    long long ff = gu.shape[0] / 2;
    Buf out = d.pool.get((size_t)n * (size_t)ff * 2);
    check(jb_gemm_tc_swiglu(a, gu.ptr, out.ptr, as_int(n, "rows"), as_int(ff, "features"), as_int(k, "width"),
                            d.stream), "linear_swiglu (tcgen05)");
    return out;
}

// ----------------------------------------------------------------- attention
Buf qk_norm_rope_append(Device &d, const Stack &qkv, const DevTensor *q_w, const DevTensor *k_w, float eps,
                        const float *cs, const float *sn, const int32_t *row_pos, const int32_t *row_seq,
                        const AttnCache &c, const AttnGeometry &g, DType out_dt) {
    long long width = (long long)(g.nh + 2 * g.nkv) * g.hd;
    if (qkv.m != width) fail(JB_LLM_EINVAL, "qk_norm_rope_append: qkv is not heads + 2 kv_heads wide");
    int w_dt = 0;
    if (q_w) {
        if (!k_w || q_w->dt != k_w->dt || q_w->numel() != g.hd || k_w->numel() != g.hd)
            fail(JB_LLM_EINVAL, "qk_norm_rope_append: q and k norm weights of one type and the head's size");
        need_float(q_w->dt, "q_norm weight");
        w_dt = q_w->dt;
    }
    bool append = c.writes && c.k != nullptr;
    if (append && c.dt != out_dt) fail(JB_LLM_EINVAL, "qk_norm_rope_append: the cache is of another type");
    Buf q = d.pool.get((size_t)qkv.n * (size_t)g.nh * (size_t)g.hd * dtype_size(out_dt));
    check(jb_qk_norm_rope_append(qkv.data(), qkv.S, qkv.stride(), q_w ? q_w->ptr : nullptr,
                                 k_w ? k_w->ptr : nullptr, w_dt, eps, cs, sn, cs ? g.hd / 2 : 0, row_pos,
                                 row_seq, c.block_table, c.bt_stride, q.ptr, append ? c.k : nullptr,
                                 append ? c.v : nullptr, out_dt, as_int(qkv.n, "rows"), g.nh, g.nkv, g.hd,
                                 d.stream), "qk_norm_rope_append");
    return q;
}

int attention_block_positions(int nh, int nkv) { return jb_attn_tc_block_positions(nh, nkv); }
bool attention_tc_ok(int nh, int nkv, int hd) { return jb_attn_tc_ok(nh, nkv, hd) != 0; }

Buf attention_blocks(Device &d, const long long *row0, const long long *pos0, const long long *len,
                     int n_seqs, int per, int *n_blocks) {
    struct B { int32_t row, count, pos, seq; };
    std::vector<B> rows;
    for (int i = 0; i < n_seqs; i++)
        for (long long a = 0; a < len[i]; a += per)
            rows.push_back({(int32_t)(row0[i] + a), (int32_t)std::min<long long>(per, len[i] - a),
                            (int32_t)(pos0[i] + a), (int32_t)i});
    // the runs that end latest see the most keys and take longest: they start first
    std::stable_sort(rows.begin(), rows.end(),
                     [](const B &x, const B &y) { return x.pos + x.count > y.pos + y.count; });
    *n_blocks = (int)rows.size();
    Buf out = d.pool.get(std::max<size_t>(rows.size() * sizeof(B), 16));
    d.upload(out.ptr, rows.data(), rows.size() * sizeof(B));
    return out;
}

// Into how many CTAs the chunks of one (token, KV head) pair are cut.  A CTA costs
// about three chunks' time to set up, and CTAs beyond the device's places (two per
// SM) come in waves: the cut that finishes first by that estimate.
static int decode_parts(long long pairs, int chunks, int places) {
    int best = 1;
    double best_t = -1;
    for (int parts = 1; parts <= chunks; parts++) {
        int per_cta = (chunks + parts - 1) / parts;
        long long ctas = pairs * ((chunks + per_cta - 1) / per_cta);
        long long waves = (ctas + places - 1) / places;
        double t = (double)waves * (3.0 + per_cta);
        if (best_t < 0 || t < best_t) { best = parts; best_t = t; }
    }
    return best;
}

static const size_t ATT_SCRATCH_BYTES = (size_t)256 << 20;

Buf attention(Device &d, const void *q, long long n, const AttnCache &c, const AttnGeometry &g,
              const int32_t *row_pos, const int32_t *row_seq, int max_chunks, const int32_t *blocks,
              int n_blocks, bool decode, bool force_simt, bool head_major) {
    need_float(c.dt, "attention");
    int ni = as_int(n, "rows");
    int vd = g.value_dim();
    Buf out = d.pool.get((size_t)n * (size_t)g.nh * (size_t)vd * dtype_size(c.dt));
    bool tc = !force_simt && vd == g.hd && c.dt == BF16 && (decode || blocks != nullptr) &&
              !c.v_ld && !head_major && attention_tc_ok(g.nh, g.nkv, g.hd) &&
              (decode || !g.head_scale || g.head_scale_positive);
    // kept first tokens and weights that are sigmoids: the prefill kernel has them for all its
    // sizes, of the decode kernels the one that runs over several chunks
    bool special = g.keep_first || g.score_bias;
    if (tc && special && ((decode && !jb_attn_tc_decode_runs(g.nh, g.nkv, g.hd)) ||
                          (g.score_bias && (g.head_scale || g.sink || g.softcap != 0.0f || g.slopes))))
        tc = false;
    if (tc && !decode) {
        check(jb_attn_tc_prefill_gen(q, c.k, c.v, c.n_pages, blocks, n_blocks, c.block_table, c.bt_stride,
                                     out.ptr, ni, g.nh, g.nkv, g.hd, g.window, g.scale, g.head_scale,
                                     g.sink, g.softcap, g.slopes, g.keep_first, g.score_bias, d.stream),
              "attention (tcgen05, prefill)");
        return out;
    }
    int parts = max_chunks, per_cta = 1;
    int kc = attention_kept_chunks(g.window, g.keep_first);
    if (tc) {
        // CTAs per (token, KV head): each runs over per_cta chunks and leaves one partial;
        // the kept first tokens' chunks are a CTA and a partial each, before the others
        int win = std::max(max_chunks - kc, 1);
        parts = win;
        if (jb_attn_tc_decode_runs(g.nh, g.nkv, g.hd))
            parts = decode_parts(std::min<long long>(n, 4096) * g.nkv, win, 2 * d.sm_count);
        per_cta = (win + parts - 1) / parts;
        parts = kc + (win + per_cta - 1) / per_cta;
    }
    long long per_row = jb_attention_scratch(1, g.nh, vd, parts);
    long long rows_per_call = std::max<long long>(1, std::min<long long>(n, (long long)(ATT_SCRATCH_BYTES / 4) /
                                                                                 std::max<long long>(per_row, 1)));
    Buf scratch = d.pool.get((size_t)per_row * (size_t)rows_per_call * 4);
    for (long long row0 = 0; row0 < n; row0 += rows_per_call) {
        int cnt = (int)std::min<long long>(rows_per_call, n - row0);
        if (tc) {
            check(jb_attn_tc_decode_gen(q, c.k, c.v, c.n_pages, row_pos, row_seq, c.block_table,
                                        c.bt_stride, scratch.as<float>(), ni, (int)row0, cnt, g.nh, g.nkv,
                                        g.hd, g.window, g.scale, g.head_scale, g.softcap, g.slopes,
                                        g.keep_first, g.score_bias, std::max(max_chunks, kc + 1), per_cta,
                                        d.stream), "attention (tcgen05, decode)");
            check(jb_attention_merge_gen(scratch.as<float>(), row_pos, out.ptr, c.dt, (int)row0, cnt, g.nh,
                                         g.hd, g.window, parts, per_cta, g.sink, g.keep_first,
                                         g.score_bias ? 1 : 0, d.stream), "attention merge");
        } else {
            check(jb_attention_gen(q, c.k, c.v, c.dt, row_pos, row_seq, c.block_table, c.bt_stride,
                                   scratch.as<float>(), out.ptr, (int)row0, cnt, g.nh, g.nkv, g.hd, vd,
                                   g.window, g.scale, g.head_scale, g.sink, max_chunks, c.v_ld, g.softcap,
                                   g.slopes, head_major ? n : 0, g.keep_first, g.score_bias, d.stream),
                  "attention", 2);
        }
    }
    return out;
}

Buf attention_decode_qkv(Device &d, const Stack &qkv, const DevTensor *q_w, const DevTensor *k_w, float eps,
                         const float *cs, const float *sn, const AttnCache &c, const AttnGeometry &g,
                         const int32_t *row_pos, const int32_t *row_seq, int max_chunks, const float *bias) {
    if (c.dt != BF16 || !c.k || !jb_attn_tc_decode_runs(g.nh, g.nkv, g.hd) || g.value_dim() != g.hd ||
        g.softcap != 0.0f || g.slopes || c.v_ld)
        return Buf();
    long long width = (long long)(g.nh + (c.writes ? 2 * g.nkv : 0)) * g.hd;
    if (qkv.m < width) fail(JB_LLM_EINVAL, "attention: qkv is narrower than the heads it holds");
    int w_dt = 0;
    if (q_w) {
        if (!k_w || q_w->dt != k_w->dt) fail(JB_LLM_EINVAL, "attention: q and k norm weights of one type");
        w_dt = q_w->dt;
    }
    long long n = qkv.n;
    int ni = as_int(n, "rows");
    int parts = decode_parts(std::min<long long>(n, 4096) * g.nkv, max_chunks, 2 * d.sm_count);
    int per_cta = (max_chunks + parts - 1) / parts;
    parts = (max_chunks + per_cta - 1) / per_cta;
    long long per_row = jb_attention_scratch(1, g.nh, g.hd, parts);
    long long rows_per_call = std::max<long long>(1, std::min<long long>(n, (long long)(ATT_SCRATCH_BYTES / 4) /
                                                                                 std::max<long long>(per_row, 1)));
    Buf scratch = d.pool.get((size_t)per_row * (size_t)rows_per_call * 4);
    Buf out = d.pool.get((size_t)n * (size_t)g.nh * (size_t)g.hd * 2);
    for (long long row0 = 0; row0 < n; row0 += rows_per_call) {
        int cnt = (int)std::min<long long>(rows_per_call, n - row0);
        int code = jb_attn_tc_decode_qkv_bias(qkv.data(), qkv.S, qkv.stride(), bias, q_w ? q_w->ptr : nullptr,
                                              k_w ? k_w->ptr : nullptr, w_dt, eps, cs, sn, c.k, c.v,
                                              c.writes ? 1 : 0, c.n_pages, row_pos, row_seq, c.block_table,
                                              c.bt_stride, scratch.as<float>(), ni, (int)row0, cnt, g.nh,
                                              g.nkv, g.hd, g.window, g.scale, g.head_scale, qkv.m, max_chunks,
                                              per_cta, d.stream);
        if (code == -1 && row0 == 0) return Buf();      // an address the kernel's 16-byte loads cannot take
        check(code, "attention (tcgen05, decode, from the product's sums)");
        check(jb_attention_merge_sink(scratch.as<float>(), row_pos, out.ptr, BF16, (int)row0, cnt, g.nh, g.hd,
                                      g.window, parts, per_cta, g.sink, d.stream), "attention merge");
    }
    return out;
}

// ------------------------------------------------------------------ sampling
void sample(Device &d, const float *logits, int rows, int vocab, const SamplerArrays &s, int32_t *out) {
    if (s.temperature && !s.rng) fail(JB_LLM_EINVAL, "sample: temperature needs the random states");
    Buf chunk_keys = d.pool.get((size_t)std::max<long long>(jb_sample_scratch(rows, vocab), 1) * 8);
    int launches = jb_sample_launches(vocab, s.big_keys ? s.big_cap : 0, s.temperature != nullptr);
    check(jb_sample(logits, rows, vocab, s.row_slot, s.temperature, s.top_k, s.top_p, s.min_p, s.rng,
                    s.big_keys, s.big_probs, s.big_keys ? s.big_cap : 0,
                    (unsigned long long *)chunk_keys.ptr, out, s.forced, d.stream), "sample", launches);
}

int gemm_tc_error() { return jb_gemm_tc_error(); }
int attn_tc_error() { return jb_attn_tc_error(); }

}  // namespace ops
}  // namespace jb

// Recurrences whose state per head is a matrix: S_t = a_t S_{t-1} + b_t k_t v_t^T,
// y_t = S_t^T q_t + d v_t, with S of N x P values per head in float32, carried from step
// to step per slot.  Two mixers are instances of it:
//
//   selective state space (Mamba-2's form): per head h of H, with group g = h / (H / G)
//       dt = softplus(dt_sum + dt_bias_h);  a = exp(-exp(A_log_h) dt);  b = dt
//       k = B_g, q = C_g (N values), v = x_h (P values), d = D_h
//   linear attention with a decay per head: a = decay_h, b = 1, d = 0, k, q, v the silu of
//       the products' sums, G = H
//
// and what follows them: a gate and an RMS norm in equal parts of the row, and the sum of
// two mixers' results.  Everything here is float32: steps, decays, exponentials, the
// state, the norms.
//
// Rows are the sequences' tokens one sequence after the other (row_seq is sorted), so a
// sequence's rows are found by a search in row_seq; nothing comes from the host, and a
// captured decode step replays with other contents.
#include "common.cuh"
#include "kernels.h"

namespace jb {

struct ScanIn {
    const float *src;          // sums [S, n, ld] that hold v, k and q
    int S;
    size_t stride;
    int ld, val_col0, key_col0, qry_col0;
    int silu;                  // v, k, q are silu(sum)
    const float *dt;           // sums [dt_S, n, dt_ld] with the steps' columns, or null
    int dt_S;
    size_t dt_stride;
    int dt_ld, dt_col0;
    const float *dt_bias, *a_log, *skip;      // [H] each (with dt)
    const float *decay;                       // [H] (without dt)
};

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float sigmoid_f(float v) { return 1.0f / (1.0f + expf(-v)); }
// log(1 + e^v), the same number as the direct form wherever that does not overflow
__device__ __forceinline__ float softplus_f(float v) { return fmaxf(v, 0.0f) + log1pf(expf(-fabsf(v))); }

// first row r with row_seq[r] >= s
__device__ __forceinline__ int first_row_of(const int32_t *__restrict__ row_seq, int n, int s)
{
    int lo = 0, hi = n;
    while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if (row_seq[mid] < s)
            lo = mid + 1;
        else
            hi = mid;
    }
    return lo;
}

// A block of 128 threads per (tile of P, head, sequence).  Thread (pi, ns) holds the state
// values S[ns + i nsplit, p] of its column p in registers (up to NR of them) and walks the
// sequence's rows in order; TB rows' k, q, v, a and b are brought into shared memory
// together.  The nsplit threads of a column add their parts of y with shuffles.
// state: [H, N, P] per slot, slot_stride floats apart.  y: float32 [n, H P].
template <int NR, int TB>
__global__ void __launch_bounds__(128)
matrix_state_scan_kernel(ScanIn in, float *__restrict__ state, size_t slot_stride,
                         const int32_t *__restrict__ row_seq, const int32_t *__restrict__ seq_slot,
                         float *__restrict__ y, int n, int H, int G, int N, int P, int nsplit,
                         int every_row_starts)
{
    extern __shared__ float sm[];
    pdl_trigger();
    const int PT = 128 / nsplit;
    int tid = threadIdx.x, ns = tid % nsplit, pi = tid / nsplit;
    int p = blockIdx.x * PT + pi, h = blockIdx.y, seq = blockIdx.z;
    int g = h / (H / G);
    float *key_s = sm, *qry_s = key_s + TB * N, *val_s = qry_s + TB * N, *a_s = val_s + TB * PT, *b_s = a_s + TB;
    int r0, r1;
    if (every_row_starts) {
        r0 = seq;
        r1 = seq + 1;
    } else {
        r0 = first_row_of(row_seq, n, seq);
        r1 = first_row_of(row_seq, n, seq + 1);
    }
    if (r0 >= r1)
        return;
    float *st = state + (size_t)seq_slot[seq] * slot_stride + (size_t)h * N * P;
    bool live = p < P;
    int cnt = ns < N ? (N - ns + nsplit - 1) / nsplit : 0;
    float dskip = in.dt != nullptr && in.skip != nullptr ? in.skip[h] : 0.0f;
    float a_neg = in.dt != nullptr ? -expf(in.a_log[h]) : 0.0f;
    pdl_wait();
    float s[NR];
#pragma unroll
    for (int i = 0; i < NR; i++)
        s[i] = live && i < cnt ? st[(size_t)(ns + i * nsplit) * P + p] : 0.0f;
    for (int c0 = r0; c0 < r1; c0 += TB) {
        int tb = min(TB, r1 - c0);
        __syncthreads();
        for (int i = tid; i < tb * N; i += 128) {
            int tt = i / N, nn = i - tt * N;
            const float *row = in.src + (size_t)(c0 + tt) * in.ld;
            float kv = add_partials(0.0f, row + in.key_col0 + g * N + nn, in.S, in.stride);
            float qv = add_partials(0.0f, row + in.qry_col0 + g * N + nn, in.S, in.stride);
            key_s[i] = in.silu ? silu_f(kv) : kv;
            qry_s[i] = in.silu ? silu_f(qv) : qv;
        }
        for (int i = tid; i < tb * PT; i += 128) {
            int tt = i / PT, pp = blockIdx.x * PT + (i - tt * PT);
            float v = 0.0f;
            if (pp < P) {
                v = add_partials(0.0f, in.src + (size_t)(c0 + tt) * in.ld + in.val_col0 + h * P + pp, in.S, in.stride);
                if (in.silu)
                    v = silu_f(v);
            }
            val_s[i] = v;
        }
        if (tid < tb) {
            if (in.dt != nullptr) {
                float d = add_partials(in.dt_bias[h], in.dt + (size_t)(c0 + tid) * in.dt_ld + in.dt_col0 + h, in.dt_S,
                                       in.dt_stride);
                d = softplus_f(d);
                a_s[tid] = expf(a_neg * d);
                b_s[tid] = d;
            } else {
                a_s[tid] = in.decay[h];
                b_s[tid] = 1.0f;
            }
        }
        __syncthreads();
        for (int tt = 0; tt < tb; tt++) {
            float a = a_s[tt], v = val_s[tt * PT + pi], bv = b_s[tt] * v;
            const float *kk = key_s + tt * N + ns, *qq = qry_s + tt * N + ns;
            float acc = 0.0f;
#pragma unroll
            for (int i = 0; i < NR; i++)
                if (i < cnt) {
                    s[i] = fmaf(bv, kk[i * nsplit], a * s[i]);
                    acc = fmaf(s[i], qq[i * nsplit], acc);
                }
            for (int o = nsplit >> 1; o > 0; o >>= 1)
                acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (ns == 0 && live)
                y[(size_t)(c0 + tt) * H * P + (size_t)h * P + p] = fmaf(dskip, v, acc);
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < NR; i++)
            if (i < cnt)
                st[(size_t)(ns + i * nsplit) * P + p] = s[i];
    }
}

// out[r, c] = rms_part(y[r, :] * pre)[c] * w[c] * post, where pre = silu of the sums in
// columns pre_col0.. of `pre` (null: 1), post = sigmoid of the sums in columns post_col0..
// of `post` (null: 1), and the row is normed in `parts` equal parts, each by its own root
// mean square.  A block per (row, part).
template <typename TO>
__global__ void __launch_bounds__(256)
gated_part_norm_kernel(const float *__restrict__ y, const float *__restrict__ pre, int pre_S, size_t pre_stride,
                       int pre_ld, int pre_col0, const float *__restrict__ post, int post_S, size_t post_stride,
                       int post_ld, int post_col0, const float *__restrict__ w, float eps, TO *__restrict__ out,
                       int width, int parts)
{
    __shared__ float red[32];
    pdl_trigger();
    int r = blockIdx.x, part = blockIdx.y, len = width / parts, c0 = part * len;
    pdl_wait();
    float ss = 0.0f;
    for (int c = c0 + threadIdx.x; c < c0 + len; c += blockDim.x) {
        float v = y[(size_t)r * width + c];
        if (pre != nullptr)
            v *= silu_f(add_partials(0.0f, pre + (size_t)r * pre_ld + pre_col0 + c, pre_S, pre_stride));
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    float scale = 1.0f / sqrtf(ss / (float)len + eps);
    for (int c = c0 + threadIdx.x; c < c0 + len; c += blockDim.x) {
        float v = y[(size_t)r * width + c];
        if (pre != nullptr)
            v *= silu_f(add_partials(0.0f, pre + (size_t)r * pre_ld + pre_col0 + c, pre_S, pre_stride));
        v = (v * scale) * w[c];
        if (post != nullptr)
            v *= sigmoid_f(add_partials(0.0f, post + (size_t)r * post_ld + post_col0 + c, post_S, post_stride));
        out[(size_t)r * width + c] = from_f<TO>(v);
    }
}

// Two mixers' results as one.  wl == null: out = sl * sum(L) + sr * sum(R).  Otherwise
// out = sl * rms(sum L) wl + sr * rms(sum R) wr (each normed over the whole row).
// A block per row; out: float32 [n, m].
__global__ void __launch_bounds__(256)
pair_combine_kernel(const float *__restrict__ L, int SL, size_t strideL, const float *__restrict__ R, int SR,
                    size_t strideR, const float *__restrict__ wl, const float *__restrict__ wr, float sl, float sr,
                    float eps, float *__restrict__ out, int m)
{
    __shared__ float red[32];
    pdl_trigger();
    int r = blockIdx.x;
    pdl_wait();
    float fl = sl, fr = sr;
    if (wl != nullptr) {
        float a = 0.0f, b = 0.0f;
        for (int c = threadIdx.x; c < m; c += blockDim.x) {
            float u = add_partials(0.0f, L + (size_t)r * m + c, SL, strideL);
            float v = add_partials(0.0f, R + (size_t)r * m + c, SR, strideR);
            a = fmaf(u, u, a);
            b = fmaf(v, v, b);
        }
        a = block_sum(a, red);
        b = block_sum(b, red);
        fl = 1.0f / sqrtf(a / (float)m + eps);
        fr = 1.0f / sqrtf(b / (float)m + eps);
    }
    for (int c = threadIdx.x; c < m; c += blockDim.x) {
        float u = add_partials(0.0f, L + (size_t)r * m + c, SL, strideL);
        float v = add_partials(0.0f, R + (size_t)r * m + c, SR, strideR);
        if (wl != nullptr)
            out[(size_t)r * m + c] = sl * ((u * fl) * wl[c]) + sr * ((v * fr) * wr[c]);
        else
            out[(size_t)r * m + c] = fmaf(fl, u, fr * v);
    }
}

// g[r, j] = gelu_tanh(sum P[r, j]) * table[tokens[r], col0 + j]: a gate computed from the
// residual stream times the token's own vector for the layer.
template <typename TT, typename TO>
__global__ void __launch_bounds__(256)
token_gate_kernel(const float *__restrict__ P, int S, size_t stride, int ld, const TT *__restrict__ table,
                  int table_ld, int col0, const int32_t *__restrict__ tokens, TO *__restrict__ out, int n, int dim)
{
    pdl_trigger();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n * dim)
        return;
    int r = (int)(idx / dim), j = (int)(idx - (size_t)r * dim);
    float e = to_f(table[(size_t)tokens[r] * table_ld + col0 + j]);
    pdl_wait();
    float v = add_partials(0.0f, P + (size_t)r * ld + j, S, stride);
    float u = 0.7978845608028654f * fmaf(0.044715f * v * v, v, v);
    out[idx] = from_f<TO>(0.5f * v * (1.0f + tanhf(u)) * e);
}

}  // namespace jb

using namespace jb;

// The smallest split of N over threads that leaves at most 32 state values to a thread,
// widened while a tile of 128 / nsplit columns is more than twice P.
static int scan_nsplit(int N, int P)
{
    int ns = 1;
    while ((N + ns - 1) / ns > 32)
        ns *= 2;
    while (ns < 32 && 128 / ns >= 2 * P)
        ns *= 2;
    return ns;
}

// src: float32 [S, n, ld] holding v (H P columns from val_col0), k and q (G N columns each);
// with dt (sums [dt_S, n, dt_ld], H columns from dt_col0) the selective form, otherwise
// decay [H].  state: [H, N, P] per slot.  y: float32 [n, H P].
extern "C" int jb_matrix_state_scan(const float *src, int S, long long stride, int ld, int val_col0, int key_col0,
                                    int qry_col0, int silu, const float *dt, int dt_S, long long dt_stride,
                                    int dt_ld, int dt_col0, const float *dt_bias, const float *a_log,
                                    const float *skip, const float *decay, float *state, long long slot_stride,
                                    const int32_t *row_seq, const int32_t *seq_slot, float *y, int n, int n_seqs,
                                    int H, int G, int N, int P, int every_row_starts, cudaStream_t st)
{
    if (n <= 0 || n_seqs <= 0)
        return JB_OK;
    if (H <= 0 || G <= 0 || H % G || N <= 0 || N > 1024 || P <= 0 || S <= 0 || src == nullptr || state == nullptr ||
        y == nullptr || (dt != nullptr && (dt_bias == nullptr || a_log == nullptr || dt_S <= 0)) ||
        (dt == nullptr && decay == nullptr) || H > 65535 || n_seqs > 65535 ||
        ld < val_col0 + H * P || ld < key_col0 + G * N || ld < qry_col0 + G * N)
        return JB_EINVAL;
    int nsplit = scan_nsplit(N, P);
    if (nsplit > 32)
        return JB_EINVAL;
    constexpr int TB = 8;
    int PT = 128 / nsplit;
    ScanIn in{src, S, (size_t)stride, ld, val_col0, key_col0, qry_col0, silu, dt, dt_S, (size_t)dt_stride, dt_ld,
              dt_col0, dt_bias, a_log, skip, decay};
    dim3 grid((unsigned)((P + PT - 1) / PT), (unsigned)H, (unsigned)n_seqs);
    size_t smem = (size_t)TB * (2 * N + PT + 2) * 4;
    launch(matrix_state_scan_kernel<32, TB>, grid, 128, smem, st, in, state, (size_t)slot_stride, row_seq, seq_slot, y,
           n, H, G, N, P, nsplit, every_row_starts);
    return launch_status();
}

extern "C" int jb_gated_part_norm(const float *y, const float *pre, int pre_S, long long pre_stride, int pre_ld,
                                  int pre_col0, const float *post, int post_S, long long post_stride, int post_ld,
                                  int post_col0, const float *w, float eps, void *out, int out_dt, int n, int width,
                                  int parts, cudaStream_t st)
{
    if (n <= 0)
        return JB_OK;
    if (width <= 0 || parts <= 0 || width % parts || parts > 65535 || y == nullptr || w == nullptr ||
        (pre != nullptr && (pre_S <= 0 || pre_ld < pre_col0 + width)) ||
        (post != nullptr && (post_S <= 0 || post_ld < post_col0 + width)))
        return JB_EINVAL;
    dim3 grid((unsigned)n, (unsigned)parts);
    if (out_dt == JB_F32)
        launch(gated_part_norm_kernel<float>, grid, 256, 0, st, y, pre, pre_S, (size_t)pre_stride, pre_ld, pre_col0,
               post, post_S, (size_t)post_stride, post_ld, post_col0, w, eps, (float *)out, width, parts);
    else if (out_dt == JB_BF16)
        launch(gated_part_norm_kernel<bf16>, grid, 256, 0, st, y, pre, pre_S, (size_t)pre_stride, pre_ld, pre_col0,
               post, post_S, (size_t)post_stride, post_ld, post_col0, w, eps, (bf16 *)out, width, parts);
    else
        return JB_EINVAL;
    return launch_status();
}

extern "C" int jb_pair_combine(const float *L, int SL, long long strideL, const float *R, int SR, long long strideR,
                               const float *wl, const float *wr, float sl, float sr, float eps, float *out, int n,
                               int m, cudaStream_t st)
{
    if (n <= 0)
        return JB_OK;
    if (m <= 0 || SL <= 0 || SR <= 0 || L == nullptr || R == nullptr || out == nullptr || (wl == nullptr) != (wr == nullptr))
        return JB_EINVAL;
    launch(pair_combine_kernel, (unsigned)n, 256, 0, st, L, SL, (size_t)strideL, R, SR, (size_t)strideR, wl, wr, sl, sr,
           eps, out, m);
    return launch_status();
}

extern "C" int jb_token_gate(const float *P, int S, long long stride, int ld, const void *table, int table_dt,
                             int table_ld, int col0, const int32_t *tokens, void *out, int out_dt, int n, int dim,
                             cudaStream_t st)
{
    if (n <= 0)
        return JB_OK;
    if (dim <= 0 || ld < dim || table_ld < col0 + dim || col0 < 0 || S <= 0 || P == nullptr || table == nullptr ||
        tokens == nullptr)
        return JB_EINVAL;
    unsigned grid = (unsigned)(((size_t)n * dim + 255) / 256);
#define JB_TG(TT, TO)                                                                                          \
    launch(token_gate_kernel<TT, TO>, grid, 256, 0, st, P, S, (size_t)stride, ld, (const TT *)table, table_ld, \
           col0, tokens, (TO *)out, n, dim)
    if (table_dt == JB_F32 && out_dt == JB_F32) JB_TG(float, float);
    else if (table_dt == JB_BF16 && out_dt == JB_BF16) JB_TG(bf16, bf16);
    else if (table_dt == JB_F32 && out_dt == JB_BF16) JB_TG(float, bf16);
    else if (table_dt == JB_BF16 && out_dt == JB_F32) JB_TG(bf16, float);
    else return JB_EINVAL;
#undef JB_TG
    return launch_status();
}

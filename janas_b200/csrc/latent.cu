// Element-wise steps of latent attention, and of per-head products in general.
//
// A latent-attention mixer keeps, per position, one latent vector c [C] and one
// rotated key part kr [R] that all heads share.  Attention runs in the latent's
// own space: a head's query is carried through that head's key matrix first
// (q_lat = Wuk_h^T q_plain, [C]), the score of a key is q_lat . c + q_rot . kr, the
// weighted sum of the latents comes out [C] per head, and the head's value matrix
// is applied to that sum.  Keys and values per head are never formed.
//
// Kernels here:
//   latent_down     the down products' sums -> RMS-normed query latent (a row of
//                   activations) and the row [RMS-normed c | rotated kr] in the cache
//   latent_q_split  the query product's sums -> plain parts [H, n, D] (one head's rows
//                   together, the A operand of that head's product) and rotated parts,
//                   written at column C of the latent queries [n, H, C + R]
//   latent_q_join   the per-head products' sums [H, S, n, C] -> columns 0..C-1 of the
//                   latent queries
//   heads_gate      per-head products' sums [H, S, n, Dv] joined head by head into rows
//                   [n, H Dv], times sigmoid of a gate's sums
//   transpose_heads [H, D, C] -> [H, C, D] (a weight, once at load time)
//
// The rotation takes pairs (2i, 2i+1) of the first 2 * rot_half values by the
// angle whose cos and sin the tables hold at [position, i]; what lies beyond
// passes unchanged.  All sums, norms and angles are float32.
#include "common.cuh"
#include "kernels.h"

namespace jb {

// ONE: the products were not cut (S = 1, a prompt step): no batches of partial sums to hold,
// fewer registers, more resident blocks.
template <typename TC, bool ONE>
__global__ void __launch_bounds__(256, ONE ? 8 : 4)
latent_down_kernel(const float *__restrict__ P, int S, size_t stride, int ld, int q_col0, int q_rank,
                   const float *__restrict__ wq, int kv_col0, int kv_rank,
                   const float *__restrict__ wkv, int rot_dim, const float *__restrict__ cs,
                   const float *__restrict__ sn, int rot_half, const int32_t *__restrict__ row_pos,
                   const int32_t *__restrict__ row_seq, const int32_t *__restrict__ block_table,
                   int bt_stride, TC *__restrict__ cq_out, TC *__restrict__ k_cache,
                   TC *__restrict__ rows_out, float eps)
{
    extern __shared__ float buf[];      // q_rank + kv_rank + rot_dim sums of this row
    __shared__ float red[32];
    pdl_trigger();
    size_t row = blockIdx.x;
    int pos = row_pos[row];
    int page = block_table[(size_t)row_seq[row] * bt_stride + pos / PAGE];
    pdl_wait();
    const float *p = P + row * ld;
    float *zq = buf, *zc = buf + q_rank, *zr = zc + kv_rank;
    float sq = 0.0f, sc = 0.0f;
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) {
        float v = ONE ? p[q_col0 + i] : add_partials(0.0f, p + q_col0 + i, S, stride);
        zq[i] = v;
        sq = fmaf(v, v, sq);
    }
    for (int i = threadIdx.x; i < kv_rank + rot_dim; i += blockDim.x) {
        float v = ONE ? p[kv_col0 + i] : add_partials(0.0f, p + kv_col0 + i, S, stride);
        zc[i] = v;
        if (i < kv_rank)
            sc = fmaf(v, v, sc);
    }
    sq = block_sum(sq, red);
    sc = block_sum(sc, red);
    if (q_rank > 0) {
        float inv = 1.0f / sqrtf(sq / (float)q_rank + eps);
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
            cq_out[row * q_rank + i] = from_f<TC>(zq[i] * inv * wq[i]);
    }
    int hd = kv_rank + rot_dim;
    TC *dst = k_cache + ((size_t)page * PAGE + pos % PAGE) * hd;
    // the same row once more, beside the other rows of the step (for a step that forms
    // its keys and values per head from it), or nowhere
    TC *dst2 = rows_out != nullptr ? rows_out + row * hd : nullptr;
    float inv = 1.0f / sqrtf(sc / (float)kv_rank + eps);
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) {
        TC v = from_f<TC>(zc[i] * inv * wkv[i]);
        dst[i] = v;
        if (dst2 != nullptr)
            dst2[i] = v;
    }
    for (int i = threadIdx.x; i < rot_dim; i += blockDim.x) {
        float v = zr[i];
        if (i < 2 * rot_half) {
            float c = cs[(size_t)pos * rot_half + i / 2], s = sn[(size_t)pos * rot_half + i / 2];
            float other = zr[i ^ 1];
            v = (i & 1) ? fmaf(v, c, other * s) : fmaf(v, c, -other * s);
        }
        dst[kv_rank + i] = from_f<TC>(v);
        if (dst2 != nullptr)
            dst2[kv_rank + i] = from_f<TC>(v);
    }
}

template <typename TC>
__global__ void latent_q_split_kernel(const float *__restrict__ Q, int S, size_t stride, int nh, int D,
                                      int R, int C, const float *__restrict__ cs,
                                      const float *__restrict__ sn, int rot_half,
                                      const int32_t *__restrict__ row_pos, TC *__restrict__ q_plain,
                                      TC *__restrict__ q_lat, int n, size_t total)
{
    pdl_trigger();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total)
        return;
    int per = D + R;
    size_t row = i / ((size_t)nh * per);
    int rem = (int)(i - row * (size_t)nh * per);
    int h = rem / per, e = rem - h * per;
    int pos = row_pos[row];
    pdl_wait();
    float v = add_partials(0.0f, Q + i, S, stride);
    if (e < D) {
        // one head's rows together, or (no q_plain) the value's own place in q_lat, whose
        // rows are then [plain | rotated] and C is D
        if (q_plain != nullptr)
            q_plain[((size_t)h * n + row) * D + e] = from_f<TC>(v);
        else
            q_lat[(row * nh + h) * (size_t)(C + R) + e] = from_f<TC>(v);
        return;
    }
    int r = e - D;
    if (r < 2 * rot_half) {
        // the pair's other value, by its column within the head
        float other = add_partials(0.0f, Q + (i - e) + D + (r ^ 1), S, stride);
        float c = cs[(size_t)pos * rot_half + r / 2], s = sn[(size_t)pos * rot_half + r / 2];
        v = (r & 1) ? fmaf(v, c, other * s) : fmaf(v, c, -other * s);
    }
    q_lat[(row * nh + h) * (size_t)(C + R) + C + r] = from_f<TC>(v);
}

// p[0] + p[stride] + ... for four neighbouring values at once
__device__ __forceinline__ float4 sum4(const float *__restrict__ p, int S, size_t stride)
{
    float4 v = load4(p);
    for (int s = 1; s < S; s++) {
        float4 w = load4(p + (size_t)s * stride);
        v = make_float4(v.x + w.x, v.y + w.y, v.z + w.z, v.w + w.w);
    }
    return v;
}

// latent_q_split with four neighbouring values of a head per thread (D, R and C multiples
// of four: the four lie in the plain or in the rotated part, and hold whole pairs)
template <typename TC>
__global__ void latent_q_split_vec_kernel(const float *__restrict__ Q, int S, size_t stride, int nh, int D,
                                          int R, int C, const float *__restrict__ cs,
                                          const float *__restrict__ sn, int rot_half,
                                          const int32_t *__restrict__ row_pos, TC *__restrict__ q_plain,
                                          TC *__restrict__ q_lat, int n, size_t total4)
{
    pdl_trigger();
    size_t i4 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i4 >= total4)
        return;
    int per = D + R;
    size_t i = i4 * 4;
    size_t row = i / ((size_t)nh * per);
    int rem = (int)(i - row * (size_t)nh * per);
    int h = rem / per, e = rem - h * per;
    int pos = row_pos[row];
    pdl_wait();
    float4 v = sum4(Q + i, S, stride);
    if (e < D) {
        if (q_plain != nullptr)
            store4(q_plain + ((size_t)h * n + row) * D + e, v);
        else
            store4(q_lat + (row * nh + h) * (size_t)(C + R) + e, v);
        return;
    }
    int r = e - D;
    float o[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int u = 0; u < 4; u += 2) {
        if (r + u < 2 * rot_half) {
            float c = cs[(size_t)pos * rot_half + (r + u) / 2], s = sn[(size_t)pos * rot_half + (r + u) / 2];
            float a = o[u], b = o[u + 1];
            o[u] = fmaf(a, c, -b * s);
            o[u + 1] = fmaf(b, c, a * s);
        }
    }
    store4(q_lat + (row * nh + h) * (size_t)(C + R) + C + r, make_float4(o[0], o[1], o[2], o[3]));
}

template <typename TC>
__global__ void latent_q_join_kernel(const float *__restrict__ A, int S, int nh, int C, int R,
                                     TC *__restrict__ q_lat, int n, size_t total)
{
    pdl_trigger();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total)
        return;
    size_t row = i / ((size_t)nh * C);
    int rem = (int)(i - row * (size_t)nh * C);
    int h = rem / C, c = rem - h * C;
    pdl_wait();
    size_t one = (size_t)n * C;       // one partial sum of one head
    float v = add_partials(0.0f, A + (size_t)h * S * one + row * C + c, S, one);
    q_lat[(row * nh + h) * (size_t)(C + R) + c] = from_f<TC>(v);
}

template <typename TC>
__global__ void heads_gate_kernel(const float *__restrict__ A, int S, int nh, int Dv,
                                  const float *__restrict__ g, int Sg, size_t g_stride, int g_ld,
                                  int g_col0, TC *__restrict__ out, int n, size_t total)
{
    pdl_trigger();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total)
        return;
    int width = nh * Dv;
    size_t row = i / width;
    int col = (int)(i - row * width);
    int h = col / Dv, d = col - h * Dv;
    pdl_wait();
    size_t one = (size_t)n * Dv;
    float v = add_partials(0.0f, A + (size_t)h * S * one + row * Dv + d, S, one);
    if (g != nullptr) {
        float z = add_partials(0.0f, g + row * g_ld + g_col0 + col, Sg, g_stride);
        v *= 1.0f / (1.0f + expf(-z));
    }
    out[i] = from_f<TC>(v);
}

// out = a * sigmoid(sum of the gate's partial sums), value by value over rows [n, width]
template <typename TC>
__global__ void gate_rows_kernel(const TC *__restrict__ a, const float *__restrict__ g, int Sg,
                                 size_t g_stride, int g_ld, int g_col0, TC *__restrict__ out, int width,
                                 size_t total)
{
    pdl_trigger();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total)
        return;
    size_t row = i / width;
    int col = (int)(i - row * width);
    pdl_wait();
    float z = add_partials(0.0f, g + row * g_ld + g_col0 + col, Sg, g_stride);
    out[i] = from_f<TC>(to_f(a[i]) * (1.0f / (1.0f + expf(-z))));
}

// gate_rows with four neighbouring values per thread
template <typename TC>
__global__ void gate_rows_vec_kernel(const TC *__restrict__ a, const float *__restrict__ g, int Sg,
                                     size_t g_stride, int g_ld, int g_col0, TC *__restrict__ out, int width,
                                     size_t total4)
{
    pdl_trigger();
    size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= total4 * 4)
        return;
    size_t row = i / width;
    int col = (int)(i - row * width);
    pdl_wait();
    float4 z = sum4(g + row * g_ld + g_col0 + col, Sg, g_stride);
    float4 v = load4(a + i);
    store4(out + i, make_float4(v.x / (1.0f + expf(-z.x)), v.y / (1.0f + expf(-z.y)), v.z / (1.0f + expf(-z.z)),
                                v.w / (1.0f + expf(-z.w))));
}

template <typename T>
__global__ void transpose_heads_kernel(const T *__restrict__ in, T *__restrict__ out, int D, int C,
                                       size_t total)
{
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total)
        return;
    size_t per = (size_t)D * C;
    size_t h = i / per;
    int rem = (int)(i - h * per);
    int c = rem / D, d = rem - c * D;      // out[h][c][d] = in[h][d][c]
    out[i] = in[h * per + (size_t)d * C + c];
}

// act(sum of a product's partial sums) over the first ff columns of its rows
template <typename TO>
__global__ void activation_kernel(const float *__restrict__ z, int S, size_t stride, int ld, int kind,
                                  TO *__restrict__ out, int ff, size_t total)
{
    pdl_trigger();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total)
        return;
    size_t row = i / ff;
    int c = (int)(i - row * ff);
    pdl_wait();
    float v = add_partials(0.0f, z + row * ld + c, S, stride);
    if (kind == JB_ACT_RELU2) {
        v = fmaxf(v, 0.0f);
        v = v * v;
    } else if (kind == JB_ACT_RELU) {
        v = fmaxf(v, 0.0f);
    } else if (kind == JB_ACT_GELU_TANH) {
        float u = 0.7978845608028654f * fmaf(0.044715f * v * v, v, v);
        v = 0.5f * v * (1.0f + tanhf(u));
    } else if (kind == JB_ACT_SILU) {
        v = v / (1.0f + expf(-v));
    }
    out[i] = from_f<TO>(v);
}

__device__ __forceinline__ float act_value(float v, int kind)
{
    if (kind == JB_ACT_RELU2) {
        v = fmaxf(v, 0.0f);
        return v * v;
    }
    if (kind == JB_ACT_RELU)
        return fmaxf(v, 0.0f);
    if (kind == JB_ACT_SILU)
        return v / (1.0f + expf(-v));
    float u = 0.7978845608028654f * fmaf(0.044715f * v * v, v, v);
    return 0.5f * v * (1.0f + tanhf(u));
}

// The same, four neighbouring columns per thread, for a product that was not cut (S = 1)
// and rows and widths that are multiples of four.
template <typename TO>
__global__ void activation_vec_kernel(const float *__restrict__ z, int ld, int kind, TO *__restrict__ out,
                                      int ff, size_t total4)
{
    pdl_trigger();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total4)
        return;
    int per = ff / 4;
    size_t row = i / per;
    int c = (int)(i - row * per) * 4;
    pdl_wait();
    float4 v = load4(z + row * ld + c);
    v = make_float4(act_value(v.x, kind), act_value(v.y, kind), act_value(v.z, kind), act_value(v.w, kind));
    store4(out + row * ff + c, v);
}

}  // namespace jb

using namespace jb;

// P: the down products' sums [S, n, ld]; columns q_col0.. hold the query latent's
// q_rank values (q_rank 0: none), columns kv_col0.. the kv_rank latent values and
// then the rot_dim values of the shared key part.  cq_out [n, q_rank] and the
// cache rows [pages, 1, PAGE, kv_rank + rot_dim] are of type cache_dt.
extern "C" int jb_latent_down(const float *P, int S, long long stride, int ld, int q_col0,
                              int q_rank, const float *wq, int kv_col0, int kv_rank,
                              const float *wkv, int rot_dim, const float *cs, const float *sn,
                              int rot_half, const int32_t *row_pos, const int32_t *row_seq,
                              const int32_t *block_table, int bt_stride, void *cq_out,
                              void *k_cache, int cache_dt, int n, float eps, cudaStream_t st)
{
    return jb_latent_down_rows(P, S, stride, ld, q_col0, q_rank, wq, kv_col0, kv_rank, wkv, rot_dim, cs, sn,
                               rot_half, row_pos, row_seq, block_table, bt_stride, cq_out, k_cache,
                               nullptr, cache_dt, n, eps, st);
}

// The same; rows_out (or null): [n, kv_rank + rot_dim], the rows that go to the cache
// once more, one after the other.
extern "C" int jb_latent_down_rows(const float *P, int S, long long stride, int ld, int q_col0,
                                   int q_rank, const float *wq, int kv_col0, int kv_rank,
                                   const float *wkv, int rot_dim, const float *cs, const float *sn,
                                   int rot_half, const int32_t *row_pos, const int32_t *row_seq,
                                   const int32_t *block_table, int bt_stride, void *cq_out,
                                   void *k_cache, void *rows_out, int cache_dt, int n, float eps,
                                   cudaStream_t st)
{
    if (n <= 0)
        return JB_OK;
    if (S <= 0 || q_rank < 0 || kv_rank <= 0 || rot_dim < 0 || 2 * rot_half > rot_dim ||
        q_col0 < 0 || kv_col0 < 0 || q_col0 + q_rank > ld || kv_col0 + kv_rank + rot_dim > ld ||
        (rot_half > 0 && (cs == nullptr || sn == nullptr)) || k_cache == nullptr ||
        (q_rank > 0 && (cq_out == nullptr || wq == nullptr)) || wkv == nullptr)
        return JB_EINVAL;
    size_t smem = (size_t)(q_rank + kv_rank + rot_dim) * 4;
    if (smem > 48 * 1024)
        return JB_EINVAL;
#define JB_LD(TC, ONE)                                                                          \
    launch(latent_down_kernel<TC, ONE>, n, 256, smem, st, P, S, (size_t)stride, ld, q_col0, q_rank, wq, \
           kv_col0, kv_rank, wkv, rot_dim, cs, sn, rot_half, row_pos, row_seq, block_table,      \
           bt_stride, (TC *)cq_out, (TC *)k_cache, (TC *)rows_out, eps)
    if (cache_dt == JB_F32 && S == 1)
        JB_LD(float, true);
    else if (cache_dt == JB_F32)
        JB_LD(float, false);
    else if (cache_dt == JB_BF16 && S == 1)
        JB_LD(bf16, true);
    else if (cache_dt == JB_BF16)
        JB_LD(bf16, false);
    else
        return JB_EINVAL;
#undef JB_LD
    return launch_status();
}

// Q: the query product's sums [S, n, nh (D + R)].  q_plain: [nh, n, D]; q_lat:
// [n, nh, C + R], of which columns C.. are written here.
extern "C" int jb_latent_q_split(const float *Q, int S, long long stride, int nh, int D, int R, int C,
                                 const float *cs, const float *sn, int rot_half,
                                 const int32_t *row_pos, void *q_plain, void *q_lat, int dt, int n,
                                 cudaStream_t st)
{
    size_t total = (size_t)n * nh * (D + R);
    if (total == 0)
        return JB_OK;
    if (S <= 0 || D <= 0 || R < 0 || C <= 0 || 2 * rot_half > R ||
        (rot_half > 0 && (cs == nullptr || sn == nullptr)))
        return JB_EINVAL;
    size_t esz = dt == JB_F32 ? 4 : 2;
    if (D % 4 == 0 && R % 4 == 0 && C % 4 == 0 && stride % 4 == 0 && (uintptr_t)Q % 16 == 0 &&
        (uintptr_t)q_plain % (4 * esz) == 0 && (uintptr_t)q_lat % (4 * esz) == 0 && (dt == JB_F32 || dt == JB_BF16)) {
        size_t total4 = total / 4;
        unsigned vb = (unsigned)((total4 + 255) / 256);
        if (dt == JB_F32)
            launch(latent_q_split_vec_kernel<float>, vb, 256, 0, st, Q, S, (size_t)stride, nh, D, R, C, cs, sn,
                   rot_half, row_pos, (float *)q_plain, (float *)q_lat, n, total4);
        else
            launch(latent_q_split_vec_kernel<bf16>, vb, 256, 0, st, Q, S, (size_t)stride, nh, D, R, C, cs, sn,
                   rot_half, row_pos, (bf16 *)q_plain, (bf16 *)q_lat, n, total4);
        return launch_status();
    }
    unsigned blocks = (unsigned)((total + 255) / 256);
    if (dt == JB_F32)
        launch(latent_q_split_kernel<float>, blocks, 256, 0, st, Q, S, (size_t)stride, nh, D, R, C, cs, sn,
               rot_half, row_pos, (float *)q_plain, (float *)q_lat, n, total);
    else if (dt == JB_BF16)
        launch(latent_q_split_kernel<bf16>, blocks, 256, 0, st, Q, S, (size_t)stride, nh, D, R, C, cs, sn,
               rot_half, row_pos, (bf16 *)q_plain, (bf16 *)q_lat, n, total);
    else
        return JB_EINVAL;
    return launch_status();
}

// A: per-head products' sums [nh, S, n, C] -> columns 0 .. C-1 of q_lat [n, nh, C + R]
extern "C" int jb_latent_q_join(const float *A, int S, int nh, int C, int R, void *q_lat, int dt,
                                int n, cudaStream_t st)
{
    size_t total = (size_t)n * nh * C;
    if (total == 0)
        return JB_OK;
    if (S <= 0 || R < 0)
        return JB_EINVAL;
    unsigned blocks = (unsigned)((total + 255) / 256);
    if (dt == JB_F32)
        launch(latent_q_join_kernel<float>, blocks, 256, 0, st, A, S, nh, C, R, (float *)q_lat, n, total);
    else if (dt == JB_BF16)
        launch(latent_q_join_kernel<bf16>, blocks, 256, 0, st, A, S, nh, C, R, (bf16 *)q_lat, n, total);
    else
        return JB_EINVAL;
    return launch_status();
}

// A: per-head products' sums [nh, S, n, Dv]; g (or null): a gate's sums [Sg, n, g_ld]
// whose columns g_col0 .. g_col0 + nh Dv - 1 are the gate.  out: [n, nh Dv].
extern "C" int jb_heads_gate(const float *A, int S, int nh, int Dv, const float *g, int Sg,
                             long long g_stride, int g_ld, int g_col0, void *out, int out_dt, int n,
                             cudaStream_t st)
{
    size_t total = (size_t)n * nh * Dv;
    if (total == 0)
        return JB_OK;
    if (S <= 0 || (g != nullptr && (Sg <= 0 || g_col0 < 0 || g_col0 + nh * Dv > g_ld)))
        return JB_EINVAL;
    unsigned blocks = (unsigned)((total + 255) / 256);
    if (out_dt == JB_F32)
        launch(heads_gate_kernel<float>, blocks, 256, 0, st, A, S, nh, Dv, g, Sg, (size_t)g_stride, g_ld,
               g_col0, (float *)out, n, total);
    else if (out_dt == JB_BF16)
        launch(heads_gate_kernel<bf16>, blocks, 256, 0, st, A, S, nh, Dv, g, Sg, (size_t)g_stride, g_ld,
               g_col0, (bf16 *)out, n, total);
    else
        return JB_EINVAL;
    return launch_status();
}

// a: [n, width] of type dt; g: a gate's sums [Sg, n, g_ld] whose columns g_col0.. are the
// gate.  out [n, width] = a * sigmoid(sum g), of type dt.
extern "C" int jb_gate_rows(const void *a, const float *g, int Sg, long long g_stride, int g_ld,
                            int g_col0, void *out, int dt, int n, int width, cudaStream_t st)
{
    size_t total = (size_t)n * width;
    if (total == 0)
        return JB_OK;
    if (g == nullptr || Sg <= 0 || g_col0 < 0 || g_col0 + width > g_ld)
        return JB_EINVAL;
    size_t esz = dt == JB_F32 ? 4 : 2;
    if (width % 4 == 0 && g_ld % 4 == 0 && g_col0 % 4 == 0 && g_stride % 4 == 0 && (uintptr_t)g % 16 == 0 &&
        (uintptr_t)a % (4 * esz) == 0 && (uintptr_t)out % (4 * esz) == 0 && (dt == JB_F32 || dt == JB_BF16)) {
        size_t total4 = total / 4;
        unsigned vb = (unsigned)((total4 + 255) / 256);
        if (dt == JB_F32)
            launch(gate_rows_vec_kernel<float>, vb, 256, 0, st, (const float *)a, g, Sg, (size_t)g_stride, g_ld,
                   g_col0, (float *)out, width, total4);
        else
            launch(gate_rows_vec_kernel<bf16>, vb, 256, 0, st, (const bf16 *)a, g, Sg, (size_t)g_stride, g_ld,
                   g_col0, (bf16 *)out, width, total4);
        return launch_status();
    }
    unsigned blocks = (unsigned)((total + 255) / 256);
    if (dt == JB_F32)
        launch(gate_rows_kernel<float>, blocks, 256, 0, st, (const float *)a, g, Sg, (size_t)g_stride, g_ld,
               g_col0, (float *)out, width, total);
    else if (dt == JB_BF16)
        launch(gate_rows_kernel<bf16>, blocks, 256, 0, st, (const bf16 *)a, g, Sg, (size_t)g_stride, g_ld,
               g_col0, (bf16 *)out, width, total);
    else
        return JB_EINVAL;
    return launch_status();
}

// in [H, D, C] -> out [H, C, D], both of type dt
extern "C" int jb_transpose_heads(const void *in, void *out, int dt, int H, int D, int C, cudaStream_t st)
{
    size_t total = (size_t)H * D * C;
    if (total == 0)
        return JB_OK;
    unsigned blocks = (unsigned)((total + 255) / 256);
    if (dt == JB_F32)
        transpose_heads_kernel<float><<<blocks, 256, 0, st>>>((const float *)in, (float *)out, D, C, total);
    else if (dt == JB_BF16)
        transpose_heads_kernel<bf16><<<blocks, 256, 0, st>>>((const bf16 *)in, (bf16 *)out, D, C, total);
    else
        return JB_EINVAL;
    return launch_status();
}

// out[r, c] = act(sum_s z[s, r, c]) for c < ff; z's rows are ld long.  kind: JB_ACT_*.
extern "C" int jb_activation(const float *z, int S, long long stride, int ld, int kind, void *out,
                             int out_dt, int n, int ff, cudaStream_t st)
{
    size_t total = (size_t)n * ff;
    if (total == 0)
        return JB_OK;
    if (S <= 0 || ff > ld || kind < 0 || kind > JB_ACT_SILU)
        return JB_EINVAL;
    if (S == 1 && ff % 4 == 0 && ld % 4 == 0 && (uintptr_t)z % 16 == 0 && (uintptr_t)out % 16 == 0 &&
        (out_dt == JB_F32 || out_dt == JB_BF16)) {
        size_t total4 = total / 4;
        unsigned vb = (unsigned)((total4 + 255) / 256);
        if (out_dt == JB_F32)
            launch(activation_vec_kernel<float>, vb, 256, 0, st, z, ld, kind, (float *)out, ff, total4);
        else
            launch(activation_vec_kernel<bf16>, vb, 256, 0, st, z, ld, kind, (bf16 *)out, ff, total4);
        return launch_status();
    }
    unsigned blocks = (unsigned)((total + 255) / 256);
    if (out_dt == JB_F32)
        launch(activation_kernel<float>, blocks, 256, 0, st, z, S, (size_t)stride, ld, kind, (float *)out,
               ff, total);
    else if (out_dt == JB_BF16)
        launch(activation_kernel<bf16>, blocks, 256, 0, st, z, S, (size_t)stride, ld, kind, (bf16 *)out,
               ff, total);
    else
        return JB_EINVAL;
    return launch_status();
}

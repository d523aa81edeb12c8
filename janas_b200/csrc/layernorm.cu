// Layer norm with weight and bias over the rows of the float32 residual stream,
// with the residual add of what the layer before left fused in front of it.
//
//   x  <-  x + m * (sum_s a[s] + sum_s b[s])          (in place, when a is given)
//   out =  (x - mean) / sqrt(var + eps) * w + bias     var = mean((x - mean)^2)
//
// a and b are two stacks of partial sums (a mixer's and a feed-forward's result
// over the same input, for a layer whose sublayers run side by side); m is the
// factor on the residual branch.  One block per row; the row stays in shared
// memory between the add, the two sums and the output, so x and the partial sums
// are read once.  Mean and variance are two passes over the row in float32 (the
// variance of the deviations, not E[x^2] - mean^2), and the order of the
// additions depends only on the row's width: a row's bits are the same in any
// batch.
#include "common.cuh"
#include "kernels.h"

namespace jb {

template <typename TO>
__global__ void __launch_bounds__(256)
layernorm_kernel(float *__restrict__ x, const float *__restrict__ a, int Sa, size_t a_stride,
                 const float *__restrict__ b, int Sb, size_t b_stride, float mult,
                 const int32_t *__restrict__ row_idx, const float *__restrict__ w,
                 const float *__restrict__ bias, TO *__restrict__ out, int dm, float eps)
{
    extern __shared__ float row[];
    __shared__ float red[32];
    pdl_trigger();
    int r = blockIdx.x;
    pdl_wait();
    size_t src = row_idx != nullptr ? (size_t)row_idx[r] : (size_t)r;
    float *xr = x + src * dm;
    float sum = 0.0f;
    for (int i = threadIdx.x; i < dm; i += blockDim.x) {
        float v = xr[i];
        if (a != nullptr) {
            float d = add_partials(0.0f, a + src * dm + i, Sa, a_stride);
            if (b != nullptr)
                d += add_partials(0.0f, b + src * dm + i, Sb, b_stride);
            v = fmaf(mult, d, v);
            xr[i] = v;
        }
        row[i] = v;
        sum += v;
    }
    if (out == nullptr)
        return;
    float mean = block_sum(sum, red) / (float)dm;
    float sq = 0.0f;
    for (int i = threadIdx.x; i < dm; i += blockDim.x) {
        float d = row[i] - mean;
        sq = fmaf(d, d, sq);
    }
    float var = block_sum(sq, red) / (float)dm;
    float inv = 1.0f / sqrtf(var + eps);
    TO *o = out + (size_t)r * dm;
    for (int i = threadIdx.x; i < dm; i += blockDim.x)
        o[i] = from_f<TO>(fmaf((row[i] - mean) * inv, w[i], bias != nullptr ? bias[i] : 0.0f));
}

// The add alone, a thread per value: x += m * (sum a + sum b).  The order of the additions
// is the norm kernels' own, so a value's bits do not depend on which kernel added it.
__global__ void scaled_add_kernel(float *__restrict__ x, const float *__restrict__ a, int Sa, size_t a_stride,
                                  const float *__restrict__ b, int Sb, size_t b_stride, float mult,
                                  size_t total)
{
    pdl_trigger();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total)
        return;
    pdl_wait();
    float d = add_partials(0.0f, a + i, Sa, a_stride);
    if (b != nullptr)
        d += add_partials(0.0f, b + i, Sb, b_stride);
    x[i] = fmaf(mult, d, x[i]);
}

// The same for few rows of the bfloat16 path: a cluster of C CTAs per row, each with a
// slice of `cols` columns, so that the partial sums a decode step's products leave (many
// per value) are fetched by many threads at once.  The two sums cross the cluster through
// shared memory: every CTA writes its part into every CTA's array and adds the parts in
// rank order.
template <typename TO, int C>
__global__ void __launch_bounds__(256)
layernorm_cluster_kernel(float *__restrict__ x, const float *__restrict__ a, int Sa, size_t a_stride,
                         const float *__restrict__ b, int Sb, size_t b_stride, float mult,
                         const int32_t *__restrict__ row_idx, const float *__restrict__ w,
                         const float *__restrict__ bias, TO *__restrict__ out, int dm, int cols,
                         float eps)
{
    extern __shared__ float row[];          // this CTA's slice
    __shared__ float red[32];
    __shared__ float part_sum[C], part_sq[C];
    pdl_trigger();
    uint32_t rank = cluster_rank();
    int r = blockIdx.x / C;
    int c0 = (int)rank * cols, c1 = min(dm, c0 + cols);
    pdl_wait();
    size_t src = row_idx != nullptr ? (size_t)row_idx[r] : (size_t)r;
    float *xr = x + src * dm;
    float sum = 0.0f;
    for (int i = c0 + threadIdx.x; i < c1; i += blockDim.x) {
        float v = xr[i];
        if (a != nullptr) {
            float d = add_partials(0.0f, a + src * dm + i, Sa, a_stride);
            if (b != nullptr)
                d += add_partials(0.0f, b + src * dm + i, Sb, b_stride);
            v = fmaf(mult, d, v);
            xr[i] = v;
        }
        row[i - c0] = v;
        sum += v;
    }
    sum = block_sum(sum, red);
    if (threadIdx.x < C)
        cluster_write(&part_sum[rank], threadIdx.x, sum);
    cluster_arrive();
    cluster_wait();
    float tot = 0.0f;
#pragma unroll
    for (int k = 0; k < C; k++)
        tot += part_sum[k];
    float mean = tot / (float)dm;
    float sq = 0.0f;
    for (int i = c0 + threadIdx.x; i < c1; i += blockDim.x) {
        float d = row[i - c0] - mean;
        sq = fmaf(d, d, sq);
    }
    sq = block_sum(sq, red);
    if (threadIdx.x < C)
        cluster_write(&part_sq[rank], threadIdx.x, sq);
    cluster_arrive();
    cluster_wait();
    tot = 0.0f;
#pragma unroll
    for (int k = 0; k < C; k++)
        tot += part_sq[k];
    float inv = 1.0f / sqrtf(tot / (float)dm + eps);
    TO *o = out + (size_t)r * dm;
    for (int i = c0 + threadIdx.x; i < c1; i += blockDim.x)
        o[i] = from_f<TO>(fmaf((row[i - c0] - mean) * inv, w[i], bias != nullptr ? bias[i] : 0.0f));
}


// A norm on a sublayer's result alone, added to the residual stream:
//
//   y   = sum_s a[s] + a_bias + coef[r] * skip[r]        (the last two optional)
//   x  <- x + (y - mean y) / sqrt(var y + eps) * w + bias
//
// skip is the sublayer's own input in its storage type TS (what an identity expert of a
// routed feed-forward hands on), coef one number per row.  One block per row, the row of
// y in shared memory, two passes as above.  rms = 1: no mean is taken off (RMS norm).
template <typename TS>
__global__ void __launch_bounds__(256)
norm_residual_kernel(float *__restrict__ x, const float *__restrict__ a, int Sa, size_t a_stride,
                     const float *__restrict__ a_bias, const TS *__restrict__ skip,
                     const float *__restrict__ coef, int coef_ld, const float *__restrict__ w,
                     const float *__restrict__ bias, int dm, float eps, int rms)
{
    extern __shared__ float row[];
    __shared__ float red[32];
    pdl_trigger();
    int r = blockIdx.x;
    pdl_wait();
    float sum = 0.0f;
    float c = skip != nullptr ? coef[(size_t)r * coef_ld] : 0.0f;
    for (int i = threadIdx.x; i < dm; i += blockDim.x) {
        float v = add_partials(a_bias != nullptr ? a_bias[i] : 0.0f, a + (size_t)r * dm + i, Sa, a_stride);
        if (skip != nullptr)
            v = fmaf(c, to_f(skip[(size_t)r * dm + i]), v);
        row[i] = v;
        sum += v;
    }
    float mean = rms ? 0.0f : block_sum(sum, red) / (float)dm;
    float sq = 0.0f;
    for (int i = threadIdx.x; i < dm; i += blockDim.x) {
        float d = row[i] - mean;
        sq = fmaf(d, d, sq);
    }
    float var = block_sum(sq, red) / (float)dm;
    float inv = 1.0f / sqrtf(var + eps);
    float *xr = x + (size_t)r * dm;
    for (int i = threadIdx.x; i < dm; i += blockDim.x)
        xr[i] += fmaf((row[i] - mean) * inv, w[i], bias != nullptr ? bias[i] : 0.0f);
}

// The same for rows of up to 1024 NV values, a multiple of four, with every pointer on a
// 16-byte boundary: a thread keeps its values of the row in registers, four to a load, and
// x is read and written once.  The sums run in the same order as above within a thread.
template <typename TS, int NV>
__global__ void __launch_bounds__(256)
norm_residual_vec_kernel(float *__restrict__ x, const float *__restrict__ a, int Sa, size_t a_stride,
                         const float *__restrict__ a_bias, const TS *__restrict__ skip,
                         const float *__restrict__ coef, int coef_ld, const float *__restrict__ w,
                         const float *__restrict__ bias, int dm, float eps, int rms)
{
    __shared__ float red[32];
    pdl_trigger();
    int r = blockIdx.x;
    int nv = dm / 4;
    // the weights were there long before the kernel before this one
    float4 wv[NV];
#pragma unroll
    for (int k = 0; k < NV; k++) {
        int i = threadIdx.x + k * 256;
        wv[k] = i < nv ? load4(w + 4 * i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    pdl_wait();
    float c = skip != nullptr ? coef[(size_t)r * coef_ld] : 0.0f;
    float4 v[NV];
    float sum = 0.0f;
#pragma unroll
    for (int k = 0; k < NV; k++) {
        int i = threadIdx.x + k * 256;
        float4 t = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (i < nv) {
            if (a_bias != nullptr)
                t = load4(a_bias + 4 * i);
            const float *p = a + (size_t)r * dm + 4 * i;
            for (int sp = 0; sp < Sa; sp++) {
                float4 u = load4(p + (size_t)sp * a_stride);
                t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w;
            }
            if (skip != nullptr) {
                float4 u = load4(skip + (size_t)r * dm + 4 * i);
                t.x = fmaf(c, u.x, t.x); t.y = fmaf(c, u.y, t.y);
                t.z = fmaf(c, u.z, t.z); t.w = fmaf(c, u.w, t.w);
            }
            sum += (t.x + t.y) + (t.z + t.w);
        }
        v[k] = t;
    }
    float mean = rms ? 0.0f : block_sum(sum, red) / (float)dm;
    float sq = 0.0f;
#pragma unroll
    for (int k = 0; k < NV; k++) {
        if (threadIdx.x + k * 256 < nv) {
            float dx = v[k].x - mean, dy = v[k].y - mean, dz = v[k].z - mean, dw = v[k].w - mean;
            sq = fmaf(dx, dx, sq); sq = fmaf(dy, dy, sq); sq = fmaf(dz, dz, sq); sq = fmaf(dw, dw, sq);
        }
    }
    float var = block_sum(sq, red) / (float)dm;
    float inv = 1.0f / sqrtf(var + eps);
    float *xr = x + (size_t)r * dm;
#pragma unroll
    for (int k = 0; k < NV; k++) {
        int i = threadIdx.x + k * 256;
        if (i < nv) {
            float4 b = bias != nullptr ? load4(bias + 4 * i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            float4 o = load4(xr + 4 * i);
            o.x += fmaf((v[k].x - mean) * inv, wv[k].x, b.x);
            o.y += fmaf((v[k].y - mean) * inv, wv[k].y, b.y);
            o.z += fmaf((v[k].z - mean) * inv, wv[k].z, b.z);
            o.w += fmaf((v[k].w - mean) * inv, wv[k].w, b.w);
            store4(xr + 4 * i, o);
        }
    }
}

// The same for few rows of the bfloat16 path: a cluster of C CTAs per row (see
// layernorm_cluster_kernel).
template <typename TS, int C>
__global__ void __launch_bounds__(256)
norm_residual_cluster_kernel(float *__restrict__ x, const float *__restrict__ a, int Sa, size_t a_stride,
                             const float *__restrict__ a_bias, const TS *__restrict__ skip,
                             const float *__restrict__ coef, int coef_ld, const float *__restrict__ w,
                             const float *__restrict__ bias, int dm, int cols, float eps, int rms)
{
    extern __shared__ float row[];
    __shared__ float red[32];
    __shared__ float part_sum[C], part_sq[C];
    pdl_trigger();
    uint32_t rank = cluster_rank();
    int r = blockIdx.x / C;
    int c0 = (int)rank * cols, c1 = min(dm, c0 + cols);
    pdl_wait();
    float sum = 0.0f;
    float c = skip != nullptr ? coef[(size_t)r * coef_ld] : 0.0f;
    for (int i = c0 + threadIdx.x; i < c1; i += blockDim.x) {
        float v = add_partials(a_bias != nullptr ? a_bias[i] : 0.0f, a + (size_t)r * dm + i, Sa, a_stride);
        if (skip != nullptr)
            v = fmaf(c, to_f(skip[(size_t)r * dm + i]), v);
        row[i - c0] = v;
        sum += v;
    }
    sum = block_sum(sum, red);
    if (threadIdx.x < C)
        cluster_write(&part_sum[rank], threadIdx.x, sum);
    cluster_arrive();
    cluster_wait();
    float tot = 0.0f;
#pragma unroll
    for (int k = 0; k < C; k++)
        tot += part_sum[k];
    float mean = rms ? 0.0f : tot / (float)dm;
    float sq = 0.0f;
    for (int i = c0 + threadIdx.x; i < c1; i += blockDim.x) {
        float d = row[i - c0] - mean;
        sq = fmaf(d, d, sq);
    }
    sq = block_sum(sq, red);
    if (threadIdx.x < C)
        cluster_write(&part_sq[rank], threadIdx.x, sq);
    cluster_arrive();
    cluster_wait();
    tot = 0.0f;
#pragma unroll
    for (int k = 0; k < C; k++)
        tot += part_sq[k];
    float inv = 1.0f / sqrtf(tot / (float)dm + eps);
    float *xr = x + (size_t)r * dm;
    for (int i = c0 + threadIdx.x; i < c1; i += blockDim.x)
        xr[i] += fmaf((row[i - c0] - mean) * inv, w[i], bias != nullptr ? bias[i] : 0.0f);
}

}  // namespace jb

using namespace jb;

// x: float32 [n, dm], updated in place.  a: S stacked [n, dm] partial sums of the
// sublayer's result; a_bias: float32 [dm] or null; skip: [n, dm] of type skip_dt with
// coef (float32, one per row, coef_ld apart) or null; w, bias: float32 [dm] (bias may be
// null); rms: 1 for an RMS norm.  few_rows: a cluster of CTAs per row (the bfloat16 path's
// decode steps; the 32-bit path never sets it, so a row's bits do not depend on the batch).
extern "C" int jb_norm_residual(float *x, const float *a, int Sa, long long a_stride, const float *a_bias,
                                const void *skip, int skip_dt, const float *coef, int coef_ld,
                                const float *w, const float *bias, int n, int dm, float eps, int rms,
                                int few_rows, cudaStream_t st)
{
    if (n <= 0)
        return JB_OK;
    if (dm <= 0 || dm > 49152 / 4 || a == nullptr || Sa <= 0 || w == nullptr ||
        (skip != nullptr && (coef == nullptr || coef_ld <= 0)))
        return JB_EINVAL;
    constexpr int CL = 8;
    bool cluster = few_rows && n <= 32 && dm >= 64 * CL;
    int cols = (dm + CL - 1) / CL;
    unsigned threads = (unsigned)min(256, ((cluster ? cols : dm) + 31) / 32 * 32);
#define JB_NR(TS)                                                                                       \
    do {                                                                                                \
        if (cluster)                                                                                    \
            launch_cluster(norm_residual_cluster_kernel<TS, CL>, dim3((unsigned)n * CL), threads,       \
                           (size_t)cols * 4, st, CL, x, a, Sa, (size_t)a_stride, a_bias, (const TS *)skip, \
                           coef, coef_ld, w, bias, dm, cols, eps, rms);                                 \
        else                                                                                            \
            launch(norm_residual_kernel<TS>, (unsigned)n, threads, (size_t)dm * 4, st, x, a, Sa,        \
                   (size_t)a_stride, a_bias, (const TS *)skip, coef, coef_ld, w, bias, dm, eps, rms);   \
    } while (0)
    // rows of a multiple of four values on 16-byte boundaries: the kernel that keeps a row in
    // registers (chosen by the row's size and the addresses alone, never by the batch)
    auto al16 = [](const void *p) { return ((uintptr_t)p & 15) == 0; };
    bool vec = !cluster && dm % 4 == 0 && dm <= 8192 && al16(x) && al16(a) && al16(a_bias) && al16(skip) &&
               al16(w) && al16(bias) && a_stride % 4 == 0;
#define JB_NRV(TS, NV)                                                                                  \
    launch(norm_residual_vec_kernel<TS, NV>, (unsigned)n, 256, 0, st, x, a, Sa, (size_t)a_stride, a_bias, \
           (const TS *)skip, coef, coef_ld, w, bias, dm, eps, rms)
#define JB_NRV_ANY(TS)                                                                                  \
    do {                                                                                                \
        if (dm <= 1024) JB_NRV(TS, 1);                                                                  \
        else if (dm <= 2048) JB_NRV(TS, 2);                                                             \
        else if (dm <= 4096) JB_NRV(TS, 4);                                                             \
        else JB_NRV(TS, 8);                                                                             \
    } while (0)
    if (skip != nullptr && skip_dt != JB_F32 && skip_dt != JB_BF16)
        return JB_EINVAL;
    if (vec && (skip == nullptr || skip_dt == JB_F32))
        JB_NRV_ANY(float);
    else if (vec)
        JB_NRV_ANY(bf16);
    else if (skip == nullptr || skip_dt == JB_F32)
        JB_NR(float);
    else
        JB_NR(bf16);
#undef JB_NRV_ANY
#undef JB_NRV
#undef JB_NR
    return launch_status();
}

// x: float32 [n, dm], updated in place when a is given (b only together with a).
// row_idx (n_out int32, or null): the rows to normalize; with row_idx no add is
// done.  w, bias: float32 [dm] (bias may be null).  out null: the add alone.
extern "C" int jb_layernorm(float *x, const float *a, int Sa, long long a_stride, const float *b,
                            int Sb, long long b_stride, float mult, const int32_t *row_idx,
                            const float *w, const float *bias, void *out, int out_dt, int n_out,
                            int dm, float eps, cudaStream_t st)
{
    if (n_out <= 0)
        return JB_OK;
    if (dm <= 0 || dm > 49152 / 4 || (a == nullptr && b != nullptr) || (a != nullptr && row_idx != nullptr) ||
        (out != nullptr && w == nullptr) || (a != nullptr && Sa <= 0) || (b != nullptr && Sb <= 0))
        return JB_EINVAL;
    if (out == nullptr && a != nullptr) {
        size_t total = (size_t)n_out * dm;
        launch(scaled_add_kernel, (unsigned)((total + 255) / 256), 256, 0, st, x, a, Sa, (size_t)a_stride, b, Sb,
               (size_t)b_stride, mult, total);
        return launch_status();
    }
    // few rows of the bfloat16 path: a cluster of 8 CTAs per row (the 32-bit path keeps the
    // one kernel whatever the batch, so that a row's bits do not depend on it)
    constexpr int CL = 8;
    if (out != nullptr && out_dt == JB_BF16 && n_out <= 32 && dm >= 64 * CL) {
        int cols = (dm + CL - 1) / CL;
        unsigned th = (unsigned)min(256, (cols + 31) / 32 * 32);
        launch_cluster(layernorm_cluster_kernel<bf16, CL>, dim3((unsigned)n_out * CL), th, (size_t)cols * 4, st,
                       CL, x, a, Sa, (size_t)a_stride, b, Sb, (size_t)b_stride, mult, row_idx, w, bias,
                       (bf16 *)out, dm, cols, eps);
        return launch_status();
    }
    unsigned threads = (unsigned)min(256, (dm + 31) / 32 * 32);
    size_t smem = (size_t)dm * 4;
    if (out == nullptr || out_dt == JB_F32)
        launch(layernorm_kernel<float>, n_out, threads, smem, st, x, a, Sa, (size_t)a_stride, b, Sb,
               (size_t)b_stride, mult, row_idx, w, bias, (float *)out, dm, eps);
    else if (out_dt == JB_BF16)
        launch(layernorm_kernel<bf16>, n_out, threads, smem, st, x, a, Sa, (size_t)a_stride, b, Sb,
               (size_t)b_stride, mult, row_idx, w, bias, (bf16 *)out, dm, eps);
    else
        return JB_EINVAL;
    return launch_status();
}

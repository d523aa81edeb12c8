// A routed feed-forward's element-wise steps: the router's choice per token, and the
// experts' activation times the token's weight for each expert.
//
// The experts' up matrices lie one after the other in one matrix (then a shared
// expert's, then the router's rows), so one product over the token gives every
// expert's hidden values and the router's logits; the activation of expert e's values
// is multiplied by the token's weight for e (0 for an expert that was not chosen), and
// one down product over all experts' values at once is then the weighted sum of the
// chosen experts' outputs.  Nothing is gathered or scattered and no count reaches the
// host, so a step's launches are the same whatever the router chooses.
#include "common.cuh"
#include "kernels.h"

namespace jb {

// first index of the largest value among the lanes' (value, index) pairs
__device__ __forceinline__ void warp_argmax(float &v, int &i)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, v, o);
        int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (ov > v || (ov == v && oi < i)) {
            v = ov;
            i = oi;
        }
    }
}

// One warp per token.  logits: columns col0 .. col0 + E - 1 of the sums P [S, n, ld]
// (E counts the identity experts too).  In float32:
//   s = softmax(logits);  choice = s + correction (null: none)
//   the E experts form `groups` equal groups of neighbours; a group's score is its largest
//   choice; only the `keep` best groups' experts can be chosen; the `top` largest choices
//   among them are chosen (the lower index wins a tie); weight_e = s_e * scale.
// With sigmoid_scores, s = sigmoid(logits), each on its own, instead of the softmax; with
// group_best = b > 1 a group's score is the sum of its b largest choices.
// weights: [n, E], the weight of every chosen expert and 0 for the others.  skip_coef
// [n]: the sum of the weights of the chosen experts from first_identity on (experts whose
// output is their input).  Shared memory: 2 E + groups floats per warp.
__global__ void __launch_bounds__(128)
moe_route_kernel(const float *__restrict__ P, int S, size_t stride, int ld, int col0,
                 const float *__restrict__ correction, float *__restrict__ weights,
                 float *__restrict__ skip_coef, int n, int E, int groups, int keep, int top,
                 int first_identity, float scale, int sigmoid_scores, int group_best)
{
    extern __shared__ float sm[];
    pdl_trigger();
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int r = blockIdx.x * (blockDim.x >> 5) + warp;
    if (r >= n)
        return;
    float *s = sm + (size_t)warp * (2 * E + groups), *choice = s + E, *gs = choice + E;
    pdl_wait();
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) {
        s[e] = add_partials(0.0f, P + (size_t)r * ld + col0 + e, S, stride);
        mx = fmaxf(mx, s[e]);
    }
    mx = warp_max(mx);
    float sum = 0.0f;
    for (int e = lane; e < E; e += 32) {
        s[e] = sigmoid_scores ? 1.0f / (1.0f + expf(-s[e])) : expf(s[e] - mx);
        sum += s[e];
    }
    sum = sigmoid_scores ? 1.0f : warp_sum(sum);
    for (int e = lane; e < E; e += 32) {
        s[e] = s[e] / sum;
        choice[e] = s[e] + (correction != nullptr ? correction[e] : 0.0f);
        weights[(size_t)r * E + e] = 0.0f;
    }
    __syncwarp();
    int per = E / groups;
    if (keep < groups) {
        for (int g = lane; g < groups; g += 32) {
            // the largest choice of the group, or the sum of its group_best largest
            float m = 0.0f, last = INFINITY;
            int last_e = -1;
            for (int k = 0; k < group_best && k < per; k++) {
                float b = -INFINITY;
                int be = -1;
                for (int e = g * per; e < (g + 1) * per; e++)
                    if ((choice[e] < last || (choice[e] == last && e > last_e)) && choice[e] > b) {
                        b = choice[e];
                        be = e;
                    }
                if (be < 0)
                    break;
                m += b;
                last = b;
                last_e = be;
            }
            gs[g] = m;
        }
        __syncwarp();
        // the keep best groups get +inf as a mark, one after the other
        for (int k = 0; k < keep; k++) {
            float v = -INFINITY;
            int i = 0x7fffffff;
            for (int g = lane; g < groups; g += 32)
                if (gs[g] != INFINITY && (gs[g] > v || i == 0x7fffffff)) {
                    v = gs[g];
                    i = g;
                }
            warp_argmax(v, i);
            if (lane == 0 && i != 0x7fffffff)
                gs[i] = INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (gs[e / per] != INFINITY)
                choice[e] = -INFINITY;
        __syncwarp();
    }
    float skip = 0.0f;
    for (int k = 0; k < top; k++) {
        float v = -INFINITY;
        int i = 0x7fffffff;
        for (int e = lane; e < E; e += 32)
            if (choice[e] > v) {
                v = choice[e];
                i = e;
            }
        warp_argmax(v, i);
        if (i == 0x7fffffff)
            break;          // fewer experts may be chosen than top asks for
        if (lane == 0) {
            float wgt = s[i] * scale;
            weights[(size_t)r * E + i] = wgt;
            if (i >= first_identity)
                skip += wgt;
            choice[i] = -INFINITY;
        }
        __syncwarp();
    }
    if (lane == 0 && skip_coef != nullptr)
        skip_coef[r] = skip;
}

__device__ __forceinline__ float act_value(float v, int kind)
{
    if (kind == JB_ACT_RELU2) {
        float t = fmaxf(v, 0.0f);
        return t * t;
    }
    if (kind == JB_ACT_RELU)
        return fmaxf(v, 0.0f);
    if (kind == JB_ACT_SILU)
        return v / (1.0f + expf(-v));
    float u = 0.7978845608028654f * fmaf(0.044715f * v * v, v, v);
    return 0.5f * v * (1.0f + tanhf(u));
}

// out[r, c] = act(sum z[r, c]) * weights[r, c / ff] for c < n_experts ff, and act(...)
// alone for the columns after them (a shared expert's).  V values per thread.
template <typename TO, int V>
__global__ void __launch_bounds__(256)
activation_weighted_kernel(const float *__restrict__ z, int S, size_t stride, int ld,
                           const float *__restrict__ weights, int w_ld, int n_experts, int ff, int kind,
                           TO *__restrict__ out, int n, int width)
{
    pdl_trigger();
    // a row of blocks per row of z: no division finds a thread's row
    int r = blockIdx.x, c = (int)(blockIdx.y * blockDim.x + threadIdx.x) * V;
    if (c >= width)
        return;
    pdl_wait();
    int e = c / ff;          // V divides ff when V > 1: the values of a thread are one expert's
    float wgt = e < n_experts ? weights[(size_t)r * w_ld + e] : 1.0f;
    float v[V];
    if (V == 4) {
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (wgt != 0.0f)
            for (int s = 0; s < S; s++) {
                float4 t = *reinterpret_cast<const float4 *>(z + (size_t)s * stride + (size_t)r * ld + c);
                acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
            }
        v[0] = acc.x; v[1 % V] = acc.y; v[2 % V] = acc.z; v[3 % V] = acc.w;
    } else {
#pragma unroll
        for (int u = 0; u < V; u++)
            v[u] = wgt != 0.0f ? add_partials(0.0f, z + (size_t)r * ld + c + u, S, stride) : 0.0f;
    }
#pragma unroll
    for (int u = 0; u < V; u++)
        v[u] = wgt != 0.0f ? act_value(v[u], kind) * wgt : 0.0f;
    if (V == 4) {
        store4<TO>(out + (size_t)r * width + c, make_float4(v[0], v[1 % V], v[2 % V], v[3 % V]));
    } else {
#pragma unroll
        for (int u = 0; u < V; u++)
            out[(size_t)r * width + c + u] = from_f<TO>(v[u]);
    }
}

// The same for experts with a gate: expert e's sums are [gate (ff) | up (ff)] in columns
// 2 e ff .. of z, and out[r, e ff + j] = act(gate_j) * up_j * weights[r, e]; out: [n, n_experts ff].
// V values per thread (V = 4: ff a multiple of four and everything on 16-byte boundaries).
template <typename TO, int V>
__global__ void __launch_bounds__(256)
gated_weighted_kernel(const float *__restrict__ z, int S, size_t stride, int ld,
                      const float *__restrict__ weights, int w_ld, int ff, int kind,
                      TO *__restrict__ out, int width)
{
    pdl_trigger();
    int r = blockIdx.x, c = (int)(blockIdx.y * blockDim.x + threadIdx.x) * V;
    if (c >= width)
        return;
    pdl_wait();
    int e = c / ff, j = c - e * ff;
    float wgt = weights[(size_t)r * w_ld + e];
    const float *src = z + (size_t)r * ld + (size_t)2 * e * ff + j;
    if (V == 4) {
        float4 g = make_float4(0.0f, 0.0f, 0.0f, 0.0f), u = g;
        if (wgt != 0.0f)
            for (int sp = 0; sp < S; sp++) {
                float4 a = load4(src + (size_t)sp * stride), b = load4(src + ff + (size_t)sp * stride);
                g.x += a.x; g.y += a.y; g.z += a.z; g.w += a.w;
                u.x += b.x; u.y += b.y; u.z += b.z; u.w += b.w;
            }
        float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (wgt != 0.0f)
            v = make_float4(act_value(g.x, kind) * u.x * wgt, act_value(g.y, kind) * u.y * wgt,
                            act_value(g.z, kind) * u.z * wgt, act_value(g.w, kind) * u.w * wgt);
        store4<TO>(out + (size_t)r * width + c, v);
    } else {
        float v = 0.0f;
        if (wgt != 0.0f) {
            float g = add_partials(0.0f, src, S, stride), u = add_partials(0.0f, src + ff, S, stride);
            v = act_value(g, kind) * u * wgt;
        }
        out[(size_t)r * width + c] = from_f<TO>(v);
    }
}

// y[r, c] += coef[r * coef_ld] * skip[r, c]: a part's own input handed on with a weight
// per row (what identity experts give), for consumers that do not take it themselves.
template <typename TS>
__global__ void __launch_bounds__(256)
add_row_scaled_kernel(float *__restrict__ y, const TS *__restrict__ skip, const float *__restrict__ coef,
                      int coef_ld, int n, int m)
{
    pdl_trigger();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n * m)
        return;
    pdl_wait();
    int r = (int)(idx / m);
    y[idx] = fmaf(coef[(size_t)r * coef_ld], to_f(skip[idx]), y[idx]);
}

}  // namespace jb

using namespace jb;

extern "C" int jb_add_row_scaled(float *y, const void *skip, int skip_dt, const float *coef, int coef_ld,
                                 int n, int m, cudaStream_t st)
{
    if (n <= 0 || m <= 0)
        return JB_OK;
    if (y == nullptr || skip == nullptr || coef == nullptr || coef_ld <= 0)
        return JB_EINVAL;
    unsigned grid = (unsigned)(((size_t)n * m + 255) / 256);
    if (skip_dt == JB_F32)
        launch(add_row_scaled_kernel<float>, grid, 256, 0, st, y, (const float *)skip, coef, coef_ld, n, m);
    else if (skip_dt == JB_BF16)
        launch(add_row_scaled_kernel<bf16>, grid, 256, 0, st, y, (const bf16 *)skip, coef, coef_ld, n, m);
    else
        return JB_EINVAL;
    return launch_status();
}

extern "C" int jb_moe_route(const float *P, int S, long long stride, int ld, int col0,
                            const float *correction, float *weights, float *skip_coef, int n, int E,
                            int groups, int keep, int top, int first_identity, float scale,
                            int sigmoid_scores, int group_best, cudaStream_t st)
{
    if (n <= 0)
        return JB_OK;
    if (E <= 0 || E > 2048 || groups <= 0 || E % groups || keep <= 0 || keep > groups || top <= 0 || top > E ||
        ld < col0 + E || S <= 0 || first_identity < 0 || group_best < 1)
        return JB_EINVAL;
    size_t smem = (size_t)4 * (2 * E + groups) * 4;
    launch(moe_route_kernel, (unsigned)((n + 3) / 4), 128, smem, st, P, S, (size_t)stride, ld, col0, correction,
           weights, skip_coef, n, E, groups, keep, top, first_identity, scale, sigmoid_scores, group_best);
    return launch_status();
}

// z: float32 [S, n, ld] whose first `width` columns are n_experts blocks of ff values and
// then columns without a weight; weights: float32 [n, w_ld].  out: [n, width] in out_dt.
extern "C" int jb_activation_weighted(const float *z, int S, long long stride, int ld, const float *weights,
                                      int w_ld, int n_experts, int ff, int kind, void *out, int out_dt, int n,
                                      int width, cudaStream_t st)
{
    if (n <= 0)
        return JB_OK;
    if (n_experts == 0)
        ff = 4;          // no weighted columns: the blocks' size only has to divide a thread's values
    if (width <= 0 || ld < width || ff <= 0 || n_experts < 0 || (long long)n_experts * ff > width ||
        (n_experts > 0 && (weights == nullptr || w_ld < n_experts)) || S <= 0 ||
        (kind != JB_ACT_RELU2 && kind != JB_ACT_RELU && kind != JB_ACT_GELU_TANH && kind != JB_ACT_SILU))
        return JB_EINVAL;
    bool vec = ff % 4 == 0 && width % 4 == 0 && ld % 4 == 0 && stride % 4 == 0 && (uintptr_t)z % 16 == 0 &&
               (uintptr_t)out % 16 == 0;
    int per_row = vec ? width / 4 : width;
    if ((per_row + 255) / 256 > 65535)
        return JB_EINVAL;
    dim3 grid((unsigned)n, (unsigned)((per_row + 255) / 256));
#define JB_AW(TO, V)                                                                                       \
    launch(activation_weighted_kernel<TO, V>, grid, 256, 0, st, z, S, (size_t)stride, ld, weights, w_ld,  \
           n_experts, ff, kind, (TO *)out, n, width)
    if (out_dt == JB_F32) {
        if (vec) JB_AW(float, 4); else JB_AW(float, 1);
    } else if (out_dt == JB_BF16) {
        if (vec) JB_AW(bf16, 4); else JB_AW(bf16, 1);
    } else {
        return JB_EINVAL;
    }
#undef JB_AW
    return launch_status();
}

// z: float32 [S, n, ld] whose first 2 n_experts ff columns are, per expert, ff gate values and
// then ff up values; weights: float32 [n, w_ld].  out: [n, n_experts ff] in out_dt.
extern "C" int jb_gated_weighted(const float *z, int S, long long stride, int ld, const float *weights, int w_ld,
                                 int n_experts, int ff, int kind, void *out, int out_dt, int n, cudaStream_t st)
{
    if (n <= 0)
        return JB_OK;
    long long width = (long long)n_experts * ff;
    if (n_experts <= 0 || ff <= 0 || ld < 2 * width || width > 0x7fffffffll || weights == nullptr || w_ld < n_experts ||
        S <= 0 || (kind != JB_ACT_RELU2 && kind != JB_ACT_RELU && kind != JB_ACT_GELU_TANH && kind != JB_ACT_SILU) ||
        (width + 255) / 256 > 65535)
        return JB_EINVAL;
    bool vec = ff % 4 == 0 && ld % 4 == 0 && stride % 4 == 0 && (uintptr_t)z % 16 == 0 && (uintptr_t)out % 16 == 0;
    long long per_row = vec ? width / 4 : width;
    dim3 grid((unsigned)n, (unsigned)((per_row + 255) / 256));
#define JB_GW(TO, V)                                                                                        \
    launch(gated_weighted_kernel<TO, V>, grid, 256, 0, st, z, S, (size_t)stride, ld, weights, w_ld, ff, kind, \
           (TO *)out, (int)width)
    if (out_dt == JB_F32) {
        if (vec) JB_GW(float, 4); else JB_GW(float, 1);
    } else if (out_dt == JB_BF16) {
        if (vec) JB_GW(bf16, 4); else JB_GW(bf16, 1);
    } else {
        return JB_EINVAL;
    }
#undef JB_GW
    return launch_status();
}

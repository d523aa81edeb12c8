// Causal grouped-query attention over the paged cache, for prefill rows and
// decode rows alike.
//
// A row (one token of one sequence, at position pos) sees the positions
// lo..pos of its own sequence, lo = max(0, pos + 1 - window) with a window and
// 0 without.  The positions are cut into chunks of ATT_CHUNK that start at
// absolute positions; one warp computes, for one (row, KV head, chunk), the
// partial softmax of every query head of the group: the largest score m, the
// sum l of exp(score - m) and the values weighted by them.  A second kernel
// merges a row's partials in chunk order.  Both steps depend only on the row's
// own position and keys, so a row's result is the same bits whether it runs in
// a whole prompt, alone as a decoded token, or beside other sequences.
//
// This is the reference's scheme (chunks at absolute positions, partial
// (m, l, sum w v), merged in chunk order: src/llm/attention.c:27-36,870-910;
// head h uses KV head h / (heads / kv heads): :874-875; score = (q . k) *
// scale: :107-118; causal and window limits: :734-739).  Its cut-off of
// weights below exp(-80) (:574-588) is left out: such a weight is under 2e-35
// of the largest one and cannot change a float result.
#include <stdio.h>

#include "common.cuh"
#include "kernels.h"
#include "no_alloc.h"

namespace jb {

constexpr int ATT_CHUNK = 128;  // positions per partial (two pages)
constexpr int ATT_GT = 4;       // query heads a warp carries at once

template <typename T> __device__ __forceinline__ void load16(const T *p, float *out);

template <> __device__ __forceinline__ void load16<float>(const float *p, float *out)
{
    const float4 *q = reinterpret_cast<const float4 *>(p);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        float4 v = q[i];
        out[4 * i + 0] = v.x;
        out[4 * i + 1] = v.y;
        out[4 * i + 2] = v.z;
        out[4 * i + 3] = v.w;
    }
}

template <> __device__ __forceinline__ void load16<bf16>(const bf16 *p, float *out)
{
    const uint4 *q = reinterpret_cast<const uint4 *>(p);
#pragma unroll
    for (int i = 0; i < 2; i++) {
        uint4 v = q[i];
        uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            out[8 * i + 2 * j + 0] = __uint_as_float(w[j] << 16);
            out[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        }
    }
}

// Up to 16 values of a head whose size is no multiple of 16 (rows of such heads
// lie at no 16-byte boundary): one by one, zeros beyond `count`.
template <typename T> __device__ __forceinline__ void load_some(const T *p, float *out, int count)
{
#pragma unroll
    for (int j = 0; j < 16; j++)
        out[j] = j < count ? to_f(p[j]) : 0.0f;
}

// Partials that the kept first tokens of a windowed mixer take: their chunks.
__host__ __device__ inline int kept_chunks(int window, int keep_first)
{
    return window > 0 && keep_first > 0 ? (keep_first + ATT_CHUNK - 1) / ATT_CHUNK : 0;
}

// Scratch per (row, head, chunk index): m, l, then hd weighted values (hd: the
// values' head size).
__host__ __device__ inline size_t part_at(size_t row, int nh, int h, int max_chunks, int ci,
                                          int hd)
{
    return ((row * nh + h) * max_chunks + ci) * (size_t)(hd + 2);
}

// LPK lanes share one key (16 values of the head each); 32 / LPK keys a step.
template <typename T, int LPK>
__global__ void __launch_bounds__(128)
attn_partial_kernel(const T *__restrict__ q, const T *__restrict__ k_cache,
                    const T *__restrict__ v_cache, const int32_t *__restrict__ row_pos,
                    const int32_t *__restrict__ row_seq, const int32_t *__restrict__ block_table,
                    int bt_stride, float *__restrict__ part, int row0, int n_rows, int nh, int nkv,
                    int hd, int vd, int window, float scale,
                    const float *__restrict__ head_scale, int max_chunks, int v_ld, float softcap,
                    const float *__restrict__ slopes, int keep_first,
                    const float *__restrict__ score_bias)
{
    constexpr int KPW = 32 / LPK;
    pdl_trigger();
    pdl_wait();
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    size_t item = (size_t)blockIdx.x * 4 + warp;
    if (item >= (size_t)n_rows * max_chunks)
        return;
    int lrow = (int)(item / max_chunks), ci = (int)(item % max_chunks);
    int row = row0 + lrow;
    int kvh = blockIdx.y;
    int group = nh / nkv;
    int g0 = blockIdx.z * ATT_GT;
    int gt = min(ATT_GT, group - g0);
    int h0 = kvh * group + g0;

    int pos = row_pos[row];
    int lo = window > 0 && pos + 1 > window ? pos + 1 - window : 0;
    // With kept first tokens the first kept_chunks(keep_first) partials of a row are
    // those tokens' chunks, as far as they lie before the window; the window's chunks
    // follow.  A partial whose range is empty is written as such (m = -inf, l = 0).
    int kc = kept_chunks(window, keep_first);
    int c, t0, t1;
    if (ci < kc) {
        c = ci;
        t0 = c * ATT_CHUNK;
        t1 = min(min(keep_first, lo) - 1, c * ATT_CHUNK + ATT_CHUNK - 1);
    } else {
        c = lo / ATT_CHUNK + ci - kc;
        if (c > pos / ATT_CHUNK)
            return;
        t0 = max(lo, c * ATT_CHUNK);
        t1 = min(pos, c * ATT_CHUNK + ATT_CHUNK - 1);
    }

    int cidx = lane % LPK, ks = lane / LPK;
    // a lane's 16 values of the keys (and q) and of the values; heads that are no
    // multiple of 16 are read value by value
    bool has_dims = cidx * 16 < hd, has_vals = cidx * 16 < vd;
    bool vec_k = hd % 16 == 0, vec_v = vd % 16 == 0 && v_ld % 16 == 0;
    int cnt_k = min(16, hd - cidx * 16), cnt_v = min(16, vd - cidx * 16);
    const int32_t *bt = block_table + (size_t)row_seq[row] * bt_stride;

    float qv[ATT_GT][16], o[ATT_GT][16], m[ATT_GT], l[ATT_GT];
#pragma unroll
    for (int g = 0; g < ATT_GT; g++) {
        m[g] = -INFINITY;
        l[g] = 0.0f;
#pragma unroll
        for (int j = 0; j < 16; j++)
            o[g][j] = qv[g][j] = 0.0f;
        if (g < gt && has_dims) {
            const T *qp = q + ((size_t)row * nh + h0 + g) * hd + cidx * 16;
            if (vec_k)
                load16<T>(qp, qv[g]);
            else
                load_some<T>(qp, qv[g], cnt_k);
        }
    }
    // a head's own factor on its scores (1 when the mixer has none)
    float hs[ATT_GT];
#pragma unroll
    for (int g = 0; g < ATT_GT; g++)
        hs[g] = head_scale != nullptr && g < gt ? head_scale[h0 + g] : 1.0f;
    // a head's slope: slope * distance is taken off the score of a key that far back
    float sl[ATT_GT];
#pragma unroll
    for (int g = 0; g < ATT_GT; g++)
        sl[g] = slopes != nullptr && g < gt ? slopes[h0 + g] : 0.0f;
    float inv_cap = softcap > 0.0f ? 1.0f / softcap : 0.0f;
    // a number per head added to the score, whose sigmoid is then the key's weight:
    // no maximum, no sum of weights
    float sb[ATT_GT];
#pragma unroll
    for (int g = 0; g < ATT_GT; g++)
        sb[g] = score_bias != nullptr && g < gt ? score_bias[h0 + g] : 0.0f;

    for (int base = t0; base <= t1; base += KPW) {
        int t = base + ks;
        bool valid = t <= t1;
        float kv[16];
#pragma unroll
        for (int j = 0; j < 16; j++)
            kv[j] = 0.0f;
        size_t at = 0;
        if (valid) {
            int page = bt[t / PAGE];
            at = ((size_t)page * nkv + kvh) * PAGE + (t % PAGE);
            if (has_dims) {
                if (vec_k)
                    load16<T>(k_cache + at * hd + cidx * 16, kv);
                else
                    load_some<T>(k_cache + at * hd + cidx * 16, kv, cnt_k);
            }
        }
        float s[ATT_GT];
#pragma unroll
        for (int g = 0; g < ATT_GT; g++) {
            float d = 0.0f;
#pragma unroll
            for (int j = 0; j < 16; j++)
                d = fmaf(qv[g][j], kv[j], d);
#pragma unroll
            for (int off = 1; off < LPK; off <<= 1)
                d += __shfl_xor_sync(0xffffffffu, d, off);
            s[g] = d * scale;
            if (head_scale != nullptr)
                s[g] *= hs[g];
            if (softcap > 0.0f)
                s[g] = softcap * tanhf(s[g] * inv_cap);
            if (slopes != nullptr)
                s[g] -= sl[g] * (float)(pos - t);
        }
        if (valid && has_vals) {
            if (vec_v)
                load16<T>(v_cache + at * v_ld + cidx * 16, kv);
            else
                load_some<T>(v_cache + at * v_ld + cidx * 16, kv, cnt_v);
        } else if (valid) {
#pragma unroll
            for (int j = 0; j < 16; j++)
                kv[j] = 0.0f;
        }
        if (valid && score_bias != nullptr) {
#pragma unroll
            for (int g = 0; g < ATT_GT; g++) {
                float p = 1.0f / (1.0f + expf(-(s[g] + sb[g])));
#pragma unroll
                for (int j = 0; j < 16; j++)
                    o[g][j] = fmaf(p, kv[j], o[g][j]);
            }
        } else if (valid) {
#pragma unroll
            for (int g = 0; g < ATT_GT; g++) {
                float mn = fmaxf(m[g], s[g]);
                float a = expf(m[g] - mn);  // 0 the first time (m = -inf)
                float p = expf(s[g] - mn);
                m[g] = mn;
                l[g] = l[g] * a + p;
#pragma unroll
                for (int j = 0; j < 16; j++)
                    o[g][j] = o[g][j] * a + p * kv[j];
            }
        }
    }

    // the 32 / LPK key groups of the warp into one
#pragma unroll
    for (int off = LPK; off < 32; off <<= 1) {
#pragma unroll
        for (int g = 0; g < ATT_GT; g++) {
            float mo = __shfl_xor_sync(0xffffffffu, m[g], off);
            float lo_ = __shfl_xor_sync(0xffffffffu, l[g], off);
            float mn = fmaxf(m[g], mo);
            float a = mn == -INFINITY ? 0.0f : expf(m[g] - mn);
            float b = mn == -INFINITY ? 0.0f : expf(mo - mn);
            if (score_bias != nullptr)
                a = b = 1.0f;           // plain sums
            l[g] = l[g] * a + lo_ * b;
            m[g] = mn;
#pragma unroll
            for (int j = 0; j < 16; j++) {
                float oo = __shfl_xor_sync(0xffffffffu, o[g][j], off);
                o[g][j] = o[g][j] * a + oo * b;
            }
        }
    }

    if (ks == 0) {
#pragma unroll
        for (int g = 0; g < ATT_GT; g++) {
            if (g >= gt)
                continue;
            float *dst = part + part_at((size_t)lrow, nh, h0 + g, max_chunks, ci, vd);
            if (lane == 0) {
                dst[0] = m[g];
                dst[1] = l[g];
            }
            if (has_vals) {
#pragma unroll
                for (int j = 0; j < 16; j++)
                    if (j < cnt_v)
                        dst[2 + cidx * 16 + j] = o[g][j];
            }
        }
    }
}

// Rows of a mixer whose keys are one row per position for all heads, with the
// values inside it (a latent: nkv = 1, v_cache = k_cache): one CTA per (row, chunk)
// brings the chunk's rows into shared memory once and serves every head from there,
// where the kernel above would fetch them once per group of four heads, key by key.
//
//   scores   thread (key j, half of the heads): q . k_j for four heads at a time, 16 bytes
//            of the key per load (rows padded by 16 bytes: no bank conflicts)
//   softmax  a warp per head: the chunk's maximum, weights and their sum
//   values   a thread per (8 value columns, four heads): sum_j p_hj k_j[columns]
//
// The partials (m, l, sum p v) have the layout of the kernel above; the merge kernel
// joins them.  bfloat16 only (the 32-bit path keeps one kernel for every kind of row).
constexpr int LD_THREADS = 256;
constexpr int LD_SMEM_MAX = 200 * 1024;     // bytes of shared memory it may be given

__global__ void __launch_bounds__(LD_THREADS)
latent_decode_kernel(const bf16 *__restrict__ q, const bf16 *__restrict__ k_cache,
                     const int32_t *__restrict__ row_pos, const int32_t *__restrict__ row_seq,
                     const int32_t *__restrict__ block_table, int bt_stride, float *__restrict__ part,
                     int row0, int nh, int hd, int vd, int window, float scale, int max_chunks)
{
    extern __shared__ __align__(16) uint8_t ld_smem[];
    const int ks = hd + 8;                                   // a key row's stride in values
    bf16 *Ks = reinterpret_cast<bf16 *>(ld_smem);            // [ATT_CHUNK][ks]
    bf16 *Qs = Ks + (size_t)ATT_CHUNK * ks;                  // [nh][hd]
    float *Ss = reinterpret_cast<float *>(Qs + (size_t)nh * hd);   // [nh][ATT_CHUNK] scores, then weights
    pdl_trigger();
    pdl_wait();
    int lrow = blockIdx.x / max_chunks, ci = blockIdx.x % max_chunks;
    int row = row0 + lrow;
    int pos = row_pos[row];
    int lo = window > 0 && pos + 1 > window ? pos + 1 - window : 0;
    int c = lo / ATT_CHUNK + ci;
    if (c > pos / ATT_CHUNK)
        return;
    int t0 = max(lo, c * ATT_CHUNK), t1 = min(pos, c * ATT_CHUNK + ATT_CHUNK - 1);
    int nk = t1 - t0 + 1;
    const int32_t *bt = block_table + (size_t)row_seq[row] * bt_stride;
    int tid = threadIdx.x;
    const int pieces = hd / 8;                               // 16-byte pieces of a row
    // the chunk's rows and the row's queries into shared memory
    for (int i = tid; i < nk * pieces; i += LD_THREADS) {
        int j = i / pieces, pc = i - j * pieces;
        int t = t0 + j;
        const bf16 *src = k_cache + ((size_t)bt[t / PAGE] * PAGE + (t % PAGE)) * hd + pc * 8;
        *reinterpret_cast<uint4 *>(Ks + (size_t)j * ks + pc * 8) = *reinterpret_cast<const uint4 *>(src);
    }
    for (int i = tid; i < nh * pieces; i += LD_THREADS)
        reinterpret_cast<uint4 *>(Qs)[i] = reinterpret_cast<const uint4 *>(q + (size_t)row * nh * hd)[i];
    __syncthreads();
    // ---- scores
    {
        int j = tid % ATT_CHUNK, half = tid / ATT_CHUNK;     // two threads per key
        int per_half = (nh + 1) / 2;
        int h_begin = half * per_half, h_end = min(nh, h_begin + per_half);
        const bf16 *kr = Ks + (size_t)j * ks;
        for (int h = h_begin; h < h_end; h += 4) {
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            if (j < nk) {
                for (int pc = 0; pc < pieces; pc++) {
                    float kv[8];
                    uint4 kw = *reinterpret_cast<const uint4 *>(kr + pc * 8);
                    uint32_t w[4] = {kw.x, kw.y, kw.z, kw.w};
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        kv[2 * e] = __uint_as_float(w[e] << 16);
                        kv[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
                    }
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        if (h + u < h_end) {
                            uint4 qw = *reinterpret_cast<const uint4 *>(Qs + (size_t)(h + u) * hd + pc * 8);
                            uint32_t x[4] = {qw.x, qw.y, qw.z, qw.w};
#pragma unroll
                            for (int e = 0; e < 4; e++) {
                                acc[u] = fmaf(__uint_as_float(x[e] << 16), kv[2 * e], acc[u]);
                                acc[u] = fmaf(__uint_as_float(x[e] & 0xffff0000u), kv[2 * e + 1], acc[u]);
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < 4; u++)
                if (h + u < h_end)
                    Ss[(size_t)(h + u) * ATT_CHUNK + j] = j < nk ? acc[u] * scale : -INFINITY;
        }
    }
    __syncthreads();
    // ---- a warp per head: maximum, weights, sum
    {
        int warp = tid >> 5, lane = tid & 31;
        for (int h = warp; h < nh; h += LD_THREADS / 32) {
            float *sr = Ss + (size_t)h * ATT_CHUNK;
            float v[ATT_CHUNK / 32], m = -INFINITY;
#pragma unroll
            for (int u = 0; u < ATT_CHUNK / 32; u++) {
                v[u] = sr[lane + 32 * u];
                m = fmaxf(m, v[u]);
            }
            m = warp_max(m);
            float l = 0.0f;
#pragma unroll
            for (int u = 0; u < ATT_CHUNK / 32; u++) {
                float p = expf(v[u] - m);          // 0 for the keys beyond the range (-inf)
                sr[lane + 32 * u] = p;
                l += p;
            }
            l = warp_sum(l);
            if (lane == 0) {
                float *dst = part + part_at((size_t)lrow, nh, h, max_chunks, ci, vd);
                dst[0] = m;
                dst[1] = l;
            }
        }
    }
    __syncthreads();
    // ---- values: the first vd entries of the same rows
    {
        int vp = vd / 8;
        int groups = (nh + 3) / 4;
        for (int item = tid; item < vp * groups; item += LD_THREADS) {
            int hg = item / vp, pc = item - hg * vp;
            int h = hg * 4;
            float acc[4][8];
#pragma unroll
            for (int u = 0; u < 4; u++)
#pragma unroll
                for (int e = 0; e < 8; e++)
                    acc[u][e] = 0.0f;
            for (int j = 0; j < nk; j++) {
                uint4 kw = *reinterpret_cast<const uint4 *>(Ks + (size_t)j * ks + pc * 8);
                uint32_t w[4] = {kw.x, kw.y, kw.z, kw.w};
                float kv[8];
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    kv[2 * e] = __uint_as_float(w[e] << 16);
                    kv[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
                }
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    float p = h + u < nh ? Ss[(size_t)(h + u) * ATT_CHUNK + j] : 0.0f;
#pragma unroll
                    for (int e = 0; e < 8; e++)
                        acc[u][e] = fmaf(p, kv[e], acc[u][e]);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                if (h + u >= nh)
                    continue;
                float *dst = part + part_at((size_t)lrow, nh, h + u, max_chunks, ci, vd) + 2 + pc * 8;
#pragma unroll
                for (int e = 0; e < 8; e++)
                    dst[e] = acc[u][e];
            }
        }
    }
}

// The same with the two products on the tensor cores (warp-level mma, bfloat16 in, float
// out), for rows of a multiple of 16 values:
//
//   scores   S[h][j] = q_h . k_j: warp w has the keys 16 w .. 16 w + 15 and every head
//   softmax  a warp per head, as above; the weights also as bfloat16 [head][key]
//   values   O[h][c] = sum_j p_hj k_j[c]: the warps share the value columns, 16 at a time
//
// Heads are padded to a multiple of 16 with rows of zeros, keys beyond the row's range are
// rows of zeros with weight 0.
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void *p)
{
    uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void *p)
{
    uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
                 "{%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(LD_THREADS)
latent_decode_mma_kernel(const bf16 *__restrict__ q, const bf16 *__restrict__ k_cache,
                         const int32_t *__restrict__ row_pos, const int32_t *__restrict__ row_seq,
                         const int32_t *__restrict__ block_table, int bt_stride,
                         float *__restrict__ part, int row0, int nh, int hd, int vd, int window,
                         float scale, int max_chunks)
{
    extern __shared__ __align__(16) uint8_t ld_smem[];
    const int ks = hd + 8;                                   // row strides, in values: 16 bytes of padding
    const int nh16 = (nh + 15) / 16 * 16;
    const int ps = ATT_CHUNK + 8;
    bf16 *Ks = reinterpret_cast<bf16 *>(ld_smem);            // [ATT_CHUNK][ks]
    bf16 *Qs = Ks + (size_t)ATT_CHUNK * ks;                  // [nh16][ks]
    bf16 *Ps = Qs + (size_t)nh16 * ks;                       // [nh16][ps] weights
    float *Ss = reinterpret_cast<float *>(Ps + (size_t)nh16 * ps);   // [nh][ATT_CHUNK] scores
    pdl_trigger();
    pdl_wait();
    int lrow = blockIdx.x / max_chunks, ci = blockIdx.x % max_chunks;
    int row = row0 + lrow;
    int pos = row_pos[row];
    int lo = window > 0 && pos + 1 > window ? pos + 1 - window : 0;
    int c = lo / ATT_CHUNK + ci;
    if (c > pos / ATT_CHUNK)
        return;
    int t0 = max(lo, c * ATT_CHUNK), t1 = min(pos, c * ATT_CHUNK + ATT_CHUNK - 1);
    int nk = t1 - t0 + 1;
    const int32_t *bt = block_table + (size_t)row_seq[row] * bt_stride;
    int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int pieces = hd / 8;
    const uint4 zero4 = make_uint4(0, 0, 0, 0);
    // asynchronous copies, all in flight at once: the chunk's rows and the queries
    auto copy16 = [](void *dst, const void *src) {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)),
                     "l"(src) : "memory");
    };
    for (int i = tid; i < ATT_CHUNK * pieces; i += LD_THREADS) {
        int j = i / pieces, pc = i - j * pieces;
        bf16 *dst = Ks + (size_t)j * ks + pc * 8;
        if (j < nk) {
            int t = t0 + j;
            copy16(dst, k_cache + ((size_t)bt[t / PAGE] * PAGE + (t % PAGE)) * hd + pc * 8);
        } else {
            *reinterpret_cast<uint4 *>(dst) = zero4;
        }
    }
    for (int i = tid; i < nh16 * pieces; i += LD_THREADS) {
        int h = i / pieces, pc = i - h * pieces;
        bf16 *dst = Qs + (size_t)h * ks + pc * 8;
        if (h < nh)
            copy16(dst, q + ((size_t)row * nh + h) * hd + pc * 8);
        else
            *reinterpret_cast<uint4 *>(dst) = zero4;
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    // ---- scores: this warp's 16 keys against 16 heads at a time
    {
        int j0 = warp * 16;
        // the lanes' rows for ldmatrix: A (heads x k) and B (keys x k, two tiles of 8 keys)
        int a_row = lane & 15, a_k = (lane >> 4) * 8;
        int b_row = (lane & 7) + (lane >> 4) * 8, b_k = ((lane >> 3) & 1) * 8;
        for (int h0 = 0; h0 < nh16; h0 += 16) {
            float acc[2][4] = {{0.0f, 0.0f, 0.0f, 0.0f}, {0.0f, 0.0f, 0.0f, 0.0f}};
            for (int k0 = 0; k0 < hd; k0 += 16) {
                uint32_t a[4], b[4];
                ldmatrix_x4(a, Qs + (size_t)(h0 + a_row) * ks + k0 + a_k);
                ldmatrix_x4(b, Ks + (size_t)(j0 + b_row) * ks + k0 + b_k);
                mma_bf16(acc[0], a, b[0], b[1]);
                mma_bf16(acc[1], a, b[2], b[3]);
            }
#pragma unroll
            for (int t = 0; t < 2; t++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    int h = h0 + (lane >> 2) + (e >> 1) * 8;
                    int j = j0 + t * 8 + (lane & 3) * 2 + (e & 1);
                    if (h < nh)
                        Ss[(size_t)h * ATT_CHUNK + j] = j < nk ? acc[t][e] * scale : -INFINITY;
                }
        }
    }
    __syncthreads();
    // ---- a warp per head: maximum, weights, sum
    for (int h = warp; h < nh16; h += LD_THREADS / 32) {
        bf16 *pr = Ps + (size_t)h * ps;
        if (h >= nh) {
            // a padding head's weights are zeros
#pragma unroll
            for (int u = 0; u < ATT_CHUNK / 32; u++)
                pr[lane + 32 * u] = __float2bfloat16_rn(0.0f);
            continue;
        }
        const float *sr = Ss + (size_t)h * ATT_CHUNK;
        float v[ATT_CHUNK / 32], m = -INFINITY;
#pragma unroll
        for (int u = 0; u < ATT_CHUNK / 32; u++) {
            v[u] = sr[lane + 32 * u];
            m = fmaxf(m, v[u]);
        }
        m = warp_max(m);
        float l = 0.0f;
#pragma unroll
        for (int u = 0; u < ATT_CHUNK / 32; u++) {
            // the weight as the product below sees it: the sum is of the rounded weights
            bf16 pb = __float2bfloat16_rn(expf(v[u] - m));
            pr[lane + 32 * u] = pb;
            l += __bfloat162float(pb);
        }
        l = warp_sum(l);
        if (lane == 0) {
            float *dst = part + part_at((size_t)lrow, nh, h, max_chunks, ci, vd);
            dst[0] = m;
            dst[1] = l;
        }
    }
    __syncthreads();
    // ---- values: 16 columns at a time per warp, 16 heads at a time
    {
        int a_row = lane & 15, a_k = (lane >> 4) * 8;
        int b_row = (lane & 7) + ((lane >> 3) & 1) * 8, b_c = (lane >> 4) * 8;
        for (int c0 = warp * 16; c0 < vd; c0 += (LD_THREADS / 32) * 16) {
            for (int h0 = 0; h0 < nh16; h0 += 16) {
                float acc[2][4] = {{0.0f, 0.0f, 0.0f, 0.0f}, {0.0f, 0.0f, 0.0f, 0.0f}};
#pragma unroll
                for (int j0 = 0; j0 < ATT_CHUNK; j0 += 16) {
                    uint32_t a[4], b[4];
                    ldmatrix_x4(a, Ps + (size_t)(h0 + a_row) * ps + j0 + a_k);
                    ldmatrix_x4_trans(b, Ks + (size_t)(j0 + b_row) * ks + c0 + b_c);
                    mma_bf16(acc[0], a, b[0], b[1]);
                    mma_bf16(acc[1], a, b[2], b[3]);
                }
#pragma unroll
                for (int t = 0; t < 2; t++)
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        int h = h0 + (lane >> 2) + (e >> 1) * 8;
                        int cc = c0 + t * 8 + (lane & 3) * 2 + (e & 1);
                        if (h < nh)
                            part[part_at((size_t)lrow, nh, h, max_chunks, ci, vd) + 2 + cc] = acc[t][e];
                    }
            }
        }
    }
}

static size_t latent_decode_mma_smem(int nh, int hd, int vd)
{
    if (hd % 16 || vd % 16 || vd > hd || nh <= 0)
        return 0;
    size_t nh16 = (size_t)(nh + 15) / 16 * 16;
    size_t bytes = (size_t)ATT_CHUNK * (hd + 8) * 2 + nh16 * (hd + 8) * 2 + nh16 * (ATT_CHUNK + 8) * 2 +
                   (size_t)nh * ATT_CHUNK * 4;
    return bytes <= (size_t)LD_SMEM_MAX ? bytes : 0;
}

// Bytes of shared memory the kernel above needs, or 0 where it does not take the sizes.
static size_t latent_decode_smem(int nh, int hd, int vd)
{
    if (hd % 8 || vd % 8 || vd > hd || nh <= 0)
        return 0;
    size_t bytes = (size_t)ATT_CHUNK * (hd + 8) * 2 + (size_t)nh * hd * 2 + (size_t)nh * ATT_CHUNK * 4;
    return bytes <= (size_t)LD_SMEM_MAX ? bytes : 0;
}

// N partials of one (row, head), fetched together, join the running (m, l, o):
// their largest maximum first, then each weighted by e^(its maximum - that), so
// that the weights do not wait for one another.  The sums run in chunk order.
template <int N>
__device__ __forceinline__ void merge_partials(const float *__restrict__ base, size_t stride,
                                               int c0, int n_chunks, int d, int hd, float &m,
                                               float &l, float &o)
{
    float mc[N], lc[N], oc[N];
#pragma unroll
    for (int u = 0; u < N; u++) {
        const float *p = base + (size_t)min(c0 + u, n_chunks - 1) * stride;
        mc[u] = p[0];
        lc[u] = p[1];
        oc[u] = d < hd ? p[2 + d] : 0.0f;
    }
    float mn = m;
#pragma unroll
    for (int u = 0; u < N; u++)
        mn = fmaxf(mn, mc[u]);
    float a = m == -INFINITY ? 0.0f : expf(m - mn);
    l *= a;
    o *= a;
#pragma unroll
    for (int u = 0; u < N; u++) {
        float w = c0 + u < n_chunks ? expf(mc[u] - mn) : 0.0f;
        l = fmaf(lc[u], w, l);
        o = fmaf(oc[u], w, o);
    }
    m = mn;
}

// One block per (row, head); thread d owns one value of the head.
template <typename T>
__global__ void attn_merge_kernel(const float *__restrict__ part,
                                  const int32_t *__restrict__ row_pos, T *__restrict__ out,
                                  int row0, int nh, int hd, int window, int max_chunks,
                                  int chunks_per_part, const float *__restrict__ sink,
                                  long long head_major_rows, int keep_first, int plain_sum)
{
    pdl_trigger();
    pdl_wait();
    int lrow = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
    int row = row0 + lrow;
    int pos = row_pos[row];
    int lo = window > 0 && pos + 1 > window ? pos + 1 - window : 0;
    // a partial covers chunks_per_part chunks; max_chunks is the partials' stride
    int n_chunks = (pos / ATT_CHUNK - lo / ATT_CHUNK + chunks_per_part) / chunks_per_part +
                   kept_chunks(window, keep_first);
    const float *base = part + part_at((size_t)lrow, nh, h, max_chunks, 0, hd);
    size_t stride = part_at(0, nh, 0, max_chunks, 1, hd);
    if (plain_sum) {
        // weights that are not normalized over the keys: the partials' sums, in chunk order
        float acc = 0.0f;
        if (d < hd) {
            for (int c0 = 0; c0 < n_chunks; c0++)
                acc += base[(size_t)c0 * stride + 2 + d];
            if (head_major_rows > 0)
                out[((size_t)h * head_major_rows + row) * hd + d] = from_f<T>(acc);
            else
                out[((size_t)row * nh + h) * hd + d] = from_f<T>(acc);
        }
        return;
    }
    float m = -INFINITY, l = 0.0f, o = 0.0f;
    // a row with few partials fetches four at a time, one with more sixteen, one
    // with many thirty-two: most rows need one trip to memory
    if (n_chunks <= 4) {
        merge_partials<4>(base, stride, 0, n_chunks, d, hd, m, l, o);
    } else if (n_chunks <= 16) {
        merge_partials<16>(base, stride, 0, n_chunks, d, hd, m, l, o);
    } else {
        for (int c0 = 0; c0 < n_chunks; c0 += 32)
            merge_partials<32>(base, stride, c0, n_chunks, d, hd, m, l, o);
    }
    if (sink != nullptr) {
        // a head's sink: one more term exp(sink) in the denominator, with no value
        float sk = sink[h];
        float mn = fmaxf(m, sk);
        float a = expf(m - mn);
        l = fmaf(l, a, expf(sk - mn));
        o *= a;
    }
    // head_major_rows > 0: out is [nh, that many rows, hd], one head's rows together
    if (d < hd && head_major_rows > 0)
        out[((size_t)h * head_major_rows + row) * hd + d] = from_f<T>(o / l);
    else if (d < hd)
        out[((size_t)row * nh + h) * hd + d] = from_f<T>(o / l);
}

template <typename T>
static int attention_typed(const T *q, const T *k_cache, const T *v_cache, const int32_t *row_pos,
                           const int32_t *row_seq, const int32_t *block_table, int bt_stride,
                           float *part, T *out, int row0, int n_rows, int nh, int nkv, int hd,
                           int vd, int window, float scale, const float *head_scale,
                           const float *sink, int max_chunks, int v_ld, float softcap,
                           const float *slopes, long long head_major_rows, int keep_first,
                           const float *score_bias, cudaStream_t st)
{
    int lpk = 1;
    while (lpk * 16 < max(hd, vd))
        lpk <<= 1;
    int group = nh / nkv;
    size_t items = (size_t)n_rows * max_chunks;
    dim3 grid((unsigned)((items + 3) / 4), nkv, (group + ATT_GT - 1) / ATT_GT);
#define JB_ATT(L)                                                                            \
    launch(attn_partial_kernel<T, L>, grid, 128, 0, st, q, k_cache, v_cache, row_pos, row_seq, \
           block_table, bt_stride, part, row0, n_rows, nh, nkv, hd, vd, window, scale,        \
           head_scale, max_chunks, v_ld, softcap, slopes, keep_first, score_bias)
    switch (lpk) {
    case 1: JB_ATT(1); break;
    case 2: JB_ATT(2); break;
    case 4: JB_ATT(4); break;
    case 8: JB_ATT(8); break;
    case 16: JB_ATT(16); break;
    case 32: JB_ATT(32); break;
    default: return JB_EINVAL;
    }
#undef JB_ATT
    if (cudaGetLastError() != cudaSuccess)
        return JB_ELAUNCH;
    launch(attn_merge_kernel<T>, dim3(n_rows, nh), (vd + 31) / 32 * 32, 0, st, (const float *)part,
           row_pos, out, row0, nh, vd, window, max_chunks, 1, sink, head_major_rows, keep_first,
           score_bias != nullptr ? 1 : 0);
    return launch_status();
}

}  // namespace jb

using namespace jb;

extern "C" int jb_attention_chunk() { return ATT_CHUNK; }

// Floats of scratch that n_rows rows need.
extern "C" long long jb_attention_scratch(int n_rows, int nh, int hd, int max_chunks)
{
    return (long long)part_at((size_t)n_rows, nh, 0, max_chunks, 0, hd);
}

// Rows row0 .. row0 + n_rows - 1 of the step.  q and out: [n, nh, hd]; the
// scratch holds the partials of these rows only.  max_chunks: the most chunks
// any of the rows sees.
extern "C" int jb_attention(const void *q, const void *k_cache, const void *v_cache, int dt,
                            const int32_t *row_pos, const int32_t *row_seq,
                            const int32_t *block_table, int bt_stride, float *scratch, void *out,
                            int row0, int n_rows, int nh, int nkv, int hd, int window, float scale,
                            int max_chunks, cudaStream_t st)
{
    if (hd % 16)
        return JB_EINVAL;
    return jb_attention_sink(q, k_cache, v_cache, dt, row_pos, row_seq, block_table, bt_stride,
                             scratch, out, row0, n_rows, nh, nkv, hd, hd, window, scale, nullptr,
                             nullptr, max_chunks, st);
}

// The same with what some mixers add: values of another head size than the keys
// (vd; out is then [n, nh, vd] and the scratch is counted with vd), a factor per
// head on the scores (head_scale, float [nh], or null) and a sink per head (sink,
// float [nh], or null): exp(sink) joins the softmax's denominator once, with no
// key and no value.  Head sizes that are no multiple of 16 are read value by value.
extern "C" int jb_attention_sink(const void *q, const void *k_cache, const void *v_cache, int dt,
                                 const int32_t *row_pos, const int32_t *row_seq,
                                 const int32_t *block_table, int bt_stride, float *scratch,
                                 void *out, int row0, int n_rows, int nh, int nkv, int hd, int vd,
                                 int window, float scale, const float *head_scale,
                                 const float *sink, int max_chunks, cudaStream_t st)
{
    return jb_attention_ext(q, k_cache, v_cache, dt, row_pos, row_seq, block_table, bt_stride, scratch,
                            out, row0, n_rows, nh, nkv, hd, vd, window, scale, head_scale, sink,
                            max_chunks, 0, 0.0f, nullptr, 0, st);
}

// The same with more of what mixers ask for.  v_ld (0: vd): the length of a row of
// v_cache, for values that are the first vd entries of longer rows (a latent that is
// key and value at once: v_cache is then k_cache).  softcap > 0: a score s becomes
// softcap * tanh(s / softcap).  slopes (float [nh], or null): slopes[h] * (the row's
// position - the key's) is taken off the score, after the cap.  head_major_rows > 0:
// out is [nh, head_major_rows, vd], the rows of one head together.
extern "C" int jb_attention_ext(const void *q, const void *k_cache, const void *v_cache, int dt,
                                const int32_t *row_pos, const int32_t *row_seq,
                                const int32_t *block_table, int bt_stride, float *scratch,
                                void *out, int row0, int n_rows, int nh, int nkv, int hd, int vd,
                                int window, float scale, const float *head_scale,
                                const float *sink, int max_chunks, int v_ld, float softcap,
                                const float *slopes, long long head_major_rows, cudaStream_t st)
{
    return jb_attention_gen(q, k_cache, v_cache, dt, row_pos, row_seq, block_table, bt_stride, scratch, out,
                            row0, n_rows, nh, nkv, hd, vd, window, scale, head_scale, sink, max_chunks, v_ld,
                            softcap, slopes, head_major_rows, 0, nullptr, st);
}

// The same with two more things.  keep_first > 0 (with a window): the first keep_first
// positions of a sequence stay visible to every later row, beside the window; max_chunks
// then counts their chunks too (jb_attention_kept_chunks).  score_bias (float [nh], or
// null): a key's weight is sigmoid(score + score_bias[head]) and the weights are not
// normalized over the keys (no softmax; a sink has no meaning then).
extern "C" int jb_attention_kept_chunks(int window, int keep_first)
{
    return kept_chunks(window, keep_first);
}

extern "C" int jb_attention_gen(const void *q, const void *k_cache, const void *v_cache, int dt,
                                const int32_t *row_pos, const int32_t *row_seq,
                                const int32_t *block_table, int bt_stride, float *scratch,
                                void *out, int row0, int n_rows, int nh, int nkv, int hd, int vd,
                                int window, float scale, const float *head_scale,
                                const float *sink, int max_chunks, int v_ld, float softcap,
                                const float *slopes, long long head_major_rows, int keep_first,
                                const float *score_bias, cudaStream_t st)
{
    if (n_rows <= 0)
        return JB_OK;
    if (keep_first < 0 || (score_bias != nullptr && sink != nullptr))
        return JB_EINVAL;
    if (v_ld == 0)
        v_ld = vd;
    if (hd > 512 || hd <= 0 || vd > 512 || vd <= 0 || nkv <= 0 || nh % nkv || max_chunks <= 0 ||
        nkv > 65535 || nh > 65535 || v_ld < vd || softcap < 0.0f ||
        (head_major_rows > 0 && head_major_rows < (long long)row0 + n_rows))
        return JB_EINVAL;
    if (dt == JB_F32)
        return attention_typed<float>((const float *)q, (const float *)k_cache,
                                      (const float *)v_cache, row_pos, row_seq, block_table,
                                      bt_stride, scratch, (float *)out, row0, n_rows, nh, nkv, hd,
                                      vd, window, scale, head_scale, sink, max_chunks, v_ld, softcap,
                                      slopes, head_major_rows, keep_first, score_bias, st);
    // few rows over rows that are key and value at once for all heads: the chunk is
    // brought into shared memory once for all heads
    size_t ld_bytes = latent_decode_smem(nh, hd, vd);
    if (dt == JB_BF16 && nkv == 1 && v_cache == k_cache && v_ld == hd && head_scale == nullptr &&
        softcap == 0.0f && slopes == nullptr && ld_bytes > 0 && keep_first == 0 && score_bias == nullptr &&
        (uintptr_t)q % 16 == 0 && (uintptr_t)k_cache % 16 == 0) {
        static unsigned long long smem_allowed = 0, mma_allowed = 0;
        size_t mma_bytes = latent_decode_mma_smem(nh, hd, vd);
        // said once per device, for the most the kernels may ever ask for
        if (!allow_dynamic_smem(latent_decode_kernel, LD_SMEM_MAX, smem_allowed) ||
            !allow_dynamic_smem(latent_decode_mma_kernel, LD_SMEM_MAX, mma_allowed))
            return JB_ELAUNCH;
        if (mma_bytes > 0)
            launch(latent_decode_mma_kernel, dim3((unsigned)n_rows * max_chunks), LD_THREADS, mma_bytes, st,
                   (const bf16 *)q, (const bf16 *)k_cache, row_pos, row_seq, block_table, bt_stride, scratch,
                   row0, nh, hd, vd, window, scale, max_chunks);
        else
            launch(latent_decode_kernel, dim3((unsigned)n_rows * max_chunks), LD_THREADS, ld_bytes, st,
                   (const bf16 *)q, (const bf16 *)k_cache, row_pos, row_seq, block_table, bt_stride, scratch,
                   row0, nh, hd, vd, window, scale, max_chunks);
        if (cudaGetLastError() != cudaSuccess)
            return JB_ELAUNCH;
        launch(attn_merge_kernel<bf16>, dim3(n_rows, nh), (vd + 31) / 32 * 32, 0, st, (const float *)scratch,
               row_pos, (bf16 *)out, row0, nh, vd, window, max_chunks, 1, sink, head_major_rows, 0, 0);
        return launch_status();
    }
    if (dt == JB_BF16)
        return attention_typed<bf16>((const bf16 *)q, (const bf16 *)k_cache,
                                     (const bf16 *)v_cache, row_pos, row_seq, block_table,
                                     bt_stride, scratch, (bf16 *)out, row0, n_rows, nh, nkv, hd,
                                     vd, window, scale, head_scale, sink, max_chunks, v_ld, softcap,
                                     slopes, head_major_rows, keep_first, score_bias, st);
    return JB_EINVAL;
}

// Joins partials that are already in `scratch` (written by the tensor-core
// decode kernels) for rows row0 .. row0 + n_rows - 1.  A row has one partial per
// `chunks_per_part` chunks of its range; `max_parts` partials of room per
// (row, head).
extern "C" int jb_attention_merge(const float *scratch, const int32_t *row_pos, void *out, int dt,
                                  int row0, int n_rows, int nh, int hd, int window, int max_parts,
                                  int chunks_per_part, cudaStream_t st)
{
    return jb_attention_merge_sink(scratch, row_pos, out, dt, row0, n_rows, nh, hd, window,
                                   max_parts, chunks_per_part, nullptr, st);
}

// The same with a sink per head (float [nh], or null) joining the denominator.
extern "C" int jb_attention_merge_sink(const float *scratch, const int32_t *row_pos, void *out,
                                       int dt, int row0, int n_rows, int nh, int hd, int window,
                                       int max_parts, int chunks_per_part, const float *sink,
                                       cudaStream_t st)
{
    return jb_attention_merge_gen(scratch, row_pos, out, dt, row0, n_rows, nh, hd, window, max_parts,
                                  chunks_per_part, sink, 0, 0, st);
}

// The same for a mixer with kept first tokens (their chunks are a row's first partials, one
// chunk each, before the window's) and, with plain_sum, for weights that are not normalized
// over the keys: the partials' weighted values are added and nothing is divided.
extern "C" int jb_attention_merge_gen(const float *scratch, const int32_t *row_pos, void *out,
                                      int dt, int row0, int n_rows, int nh, int hd, int window,
                                      int max_parts, int chunks_per_part, const float *sink,
                                      int keep_first, int plain_sum, cudaStream_t st)
{
    if (n_rows <= 0)
        return JB_OK;
    if (hd <= 0 || hd > 512 || nh <= 0 || nh > 65535 || max_parts <= 0 || chunks_per_part <= 0 ||
        keep_first < 0 || (plain_sum && sink != nullptr))
        return JB_EINVAL;
    dim3 grid(n_rows, nh);
    int threads = (hd + 31) / 32 * 32;
    if (dt == JB_F32)
        launch(attn_merge_kernel<float>, grid, threads, 0, st, scratch, row_pos, (float *)out, row0,
               nh, hd, window, max_parts, chunks_per_part, sink, 0ll, keep_first, plain_sum);
    else if (dt == JB_BF16)
        launch(attn_merge_kernel<bf16>, grid, threads, 0, st, scratch, row_pos, (bf16 *)out, row0,
               nh, hd, window, max_parts, chunks_per_part, sink, 0ll, keep_first, plain_sum);
    else
        return JB_EINVAL;
    return launch_status();
}

// ------------------------------------------------------ without any allocation
// See no_alloc.h.  The partial results of jb_attention_noalloc() live here.  In
// host code this name is only a stand-in for the array: the device address is
// looked up once per device below and handed to the kernels.
static __device__ __align__(256) float g_noalloc_scratch[JB_NOALLOC_SCRATCH_FLOATS];

static thread_local char t_noalloc_error[160] = "";

extern "C" const char *jb_attention_noalloc_error(void) { return t_noalloc_error; }

extern "C" int jb_attention_noalloc(const void *q, const void *k_cache, const void *v_cache,
                                    int dt, const int32_t *row_pos, const int32_t *row_seq,
                                    const int32_t *block_table, int bt_stride, void *out, int row0,
                                    int n_rows, int nh, int nkv, int hd, int window, float scale,
                                    int max_chunks, cudaStream_t st)
{
    constexpr int MAX_DEVICES = 64;
    static float *scratch_of[MAX_DEVICES];   // the array's address on each device, once known
    t_noalloc_error[0] = 0;
    if (n_rows <= 0)
        return JB_OK;
    if (nh <= 0 || hd <= 0 || max_chunks <= 0) {
        snprintf(t_noalloc_error, sizeof t_noalloc_error, "sizes must be positive");
        return JB_EINVAL;
    }
    long long need = jb_attention_scratch(n_rows, nh, hd, max_chunks);
    if (need > JB_NOALLOC_SCRATCH_FLOATS) {
        snprintf(t_noalloc_error, sizeof t_noalloc_error,
                 "%d rows need %lld floats of scratch, the fixed array has %lld: "
                 "call with fewer rows", n_rows, need, (long long)JB_NOALLOC_SCRATCH_FLOATS);
        return JB_ETOOBIG;
    }
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
        snprintf(t_noalloc_error, sizeof t_noalloc_error, "no current device (or beyond %d)",
                 MAX_DEVICES);
        return JB_EDEVICE;
    }
    float *scratch = scratch_of[dev];
    if (scratch == nullptr) {
        // first call on this device: the device address of the array
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || p == nullptr) {
            snprintf(t_noalloc_error, sizeof t_noalloc_error,
                     "cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
            return JB_EDEVICE;
        }
        scratch = scratch_of[dev] = (float *)p;
    }
    int rc = jb_attention(q, k_cache, v_cache, dt, row_pos, row_seq, block_table, bt_stride,
                          scratch, out, row0, n_rows, nh, nkv, hd, window, scale, max_chunks, st);
    if (rc == JB_EINVAL)
        snprintf(t_noalloc_error, sizeof t_noalloc_error,
                 "the kernel does not take these sizes or types");
    else if (rc != JB_OK)
        snprintf(t_noalloc_error, sizeof t_noalloc_error, "the launch failed");
    return rc;
}

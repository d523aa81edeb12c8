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

// an asynchronous copy of BYTES (4 or 16) from global to shared memory, and the wait for all of a thread's
template <int BYTES>
__device__ __forceinline__ void copy_async(float *smem, const float *gmem)
{
    uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], %2;" ::"r"(dst), "l"(gmem), "n"(BYTES) : "memory");
}
__device__ __forceinline__ void copy_async_wait() { asm volatile("cp.async.wait_all;" ::: "memory"); }

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

// A block of 128 threads per (tile of P, head, sequence or piece of one).  A warp has
// PW = 32 / nsplit columns p of the state, consecutive in memory, and nsplit lanes to a column;
// the lanes of a column hold the rows n = (i nsplit + ns) 4 + j of it in registers (up to NR),
// so that four rows' k and q come from shared memory in one load that the lanes of a column
// share out among them.  The block walks its rows in order, TB rows' k, q, v, a and b brought
// into shared memory together (by asynchronous copies where the sums are the values themselves);
// the lanes of a column add their parts of y with shuffles.
//
// MODE 0: a sequence's rows of the step from the slot's state; y and the state are written.
// MODE 1: a piece of `piece` rows from a state of zeros: the piece's own end state goes to
//         local[z] and the product of its decays to decays[z, h] (no y).
// MODE 2: a piece from the state in local[z] (what carry_kernel left there); y is written, and
//         by a sequence's last piece the slot's state.
// With pieces, blockIdx.z counts (sequence, piece); pieces that hold no row return.
// NS: the split where it is fixed at compile time (0: nsplit_arg says it).
// state: [H, N, P] per slot, slot_stride floats apart.  y: float32 [n, H P].
template <int NR, int TB, int MODE, int NS>
__global__ void __launch_bounds__(128, NR <= 16 ? 5 : 3)
matrix_state_scan_kernel(ScanIn in, float *__restrict__ state, size_t slot_stride,
                         const int32_t *__restrict__ row_seq, const int32_t *__restrict__ seq_slot,
                         float *__restrict__ y, float *__restrict__ local, float *__restrict__ decays, int n,
                         int H, int G, int N, int P, int nsplit_arg, int every_row_starts, int piece, int pieces)
{
    extern __shared__ float4 sm4[];
    float *sm = reinterpret_cast<float *>(sm4);
    pdl_trigger();
    // NS > 0: the split is known when the kernel is compiled and every lane has exactly NR rows
    // (N = NR NS), so that the places in shared memory are constants and no row needs a check
    const int nsplit = NS > 0 ? NS : nsplit_arg;
    const int PW = 32 / nsplit, PT = 4 * PW;
    const int NP = NS > 0 ? NR * NS : (N + 4 * nsplit - 1) / (4 * nsplit) * (4 * nsplit);   // rows, padded with zeros
    const int cnt4 = NS > 0 ? NR / 4 : NP / (4 * nsplit);                    // groups of four rows a lane
    int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int ns = lane / PW, pl = warp * PW + lane % PW;
    int p = blockIdx.x * PT + pl, h = blockIdx.y;
    int seq = MODE == 0 ? blockIdx.z : blockIdx.z / pieces, pc = MODE == 0 ? 0 : blockIdx.z % pieces;
    int g = h / (H / G);
    float *key_s = sm, *qry_s = key_s + TB * NP, *val_s = qry_s + (MODE == 1 ? 0 : TB * NP), *a_s = val_s + TB * PT,
          *b_s = a_s + TB;
    int r0, r1;
    if (every_row_starts) {
        r0 = seq;
        r1 = seq + 1;
    } else {
        r0 = first_row_of(row_seq, n, seq);
        r1 = first_row_of(row_seq, n, seq + 1);
    }
    bool last_piece = true;
    if (MODE != 0) {
        // A sequence that brings fewer than two pieces' rows stays whole (its first piece has
        // all its rows), so that its sums are added in the order of the one-pass form: what
        // else the step holds then does not change a sequence's bits.
        int end = r1;
        if (r1 - r0 >= 2 * piece) {
            r0 += pc * piece;
            r1 = min(r1, r0 + piece);
        } else if (pc > 0) {
            return;
        }
        last_piece = r1 == end;
    }
    if (r0 >= r1)
        return;
    float *st = MODE == 0 ? state + (size_t)seq_slot[seq] * slot_stride + (size_t)h * N * P
                          : local + ((size_t)blockIdx.z * H + h) * N * P;
    bool live = p < P;
    float dskip = in.dt != nullptr && in.skip != nullptr ? in.skip[h] : 0.0f;
    float a_neg = in.dt != nullptr ? -expf(in.a_log[h]) : 0.0f;
    pdl_wait();
    float s[NR];
#pragma unroll
    for (int i = 0; i < NR; i++) {
        int nn = ((i >> 2) * nsplit + ns) * 4 + (i & 3);
        s[i] = MODE != 1 && live && nn < N ? st[(size_t)nn * P + p] : 0.0f;
    }
    float run = 1.0f;        // the product of the piece's decays
    // TB rows' k, q, v, a and b at a time.  Where the sums are the values themselves (one partial
    // sum, no activation) they go from memory into shared memory by asynchronous copies, all of a
    // batch in flight together, 16 bytes each where everything lies on such boundaries; otherwise
    // the threads add and activate them on the way.
    const bool direct = in.S == 1 && !in.silu;
    const float *__restrict__ src = in.src;
    const int kcol = in.key_col0 + g * N, qcol = in.qry_col0 + g * N, vcol = in.val_col0 + h * P + blockIdx.x * PT;
    const bool k16 = direct && N % 4 == 0 && in.ld % 4 == 0 && kcol % 4 == 0 && qcol % 4 == 0 &&
                     (reinterpret_cast<uintptr_t>(src) & 15) == 0;
    const bool v16 = direct && PT % 4 == 0 && P % 4 == 0 && in.ld % 4 == 0 && vcol % 4 == 0 &&
                     (reinterpret_cast<uintptr_t>(src) & 15) == 0;
    if (direct) {
        // the rows' padding beyond N is never copied over: zeros once
        for (int i = tid; i < TB * (NP - N); i += 128) {
            int tt = i / (NP - N), nn = N + i - tt * (NP - N);
            key_s[tt * NP + nn] = 0.0f;
            if (MODE != 1)
                qry_s[tt * NP + nn] = 0.0f;
        }
    }
    for (int c0 = r0; c0 < r1; c0 += TB) {
        int tb = min(TB, r1 - c0);
        __syncthreads();
        if (direct) {
            if (k16) {
                int n4 = N / 4;
                for (int i = tid; i < tb * n4; i += 128) {
                    int tt = i / n4, c4 = (i - tt * n4) * 4;
                    const float *row = src + (size_t)(c0 + tt) * in.ld + c4;
                    copy_async<16>(key_s + tt * NP + c4, row + kcol);
                    if (MODE != 1)
                        copy_async<16>(qry_s + tt * NP + c4, row + qcol);
                }
            } else {
                for (int i = tid; i < tb * N; i += 128) {
                    int tt = i / N, nn = i - tt * N;
                    const float *row = src + (size_t)(c0 + tt) * in.ld + nn;
                    copy_async<4>(key_s + tt * NP + nn, row + kcol);
                    if (MODE != 1)
                        copy_async<4>(qry_s + tt * NP + nn, row + qcol);
                }
            }
            if (v16) {
                int p4 = PT / 4;
                for (int i = tid; i < tb * p4; i += 128) {
                    int tt = i / p4, c4 = (i - tt * p4) * 4;
                    if (blockIdx.x * PT + c4 < P)
                        copy_async<16>(val_s + tt * PT + c4, src + (size_t)(c0 + tt) * in.ld + vcol + c4);
                    else
                        *reinterpret_cast<float4 *>(val_s + tt * PT + c4) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                }
            } else {
                for (int i = tid; i < tb * PT; i += 128) {
                    int tt = i / PT, pp = i - tt * PT;
                    if (blockIdx.x * PT + pp < P)
                        copy_async<4>(val_s + i, src + (size_t)(c0 + tt) * in.ld + vcol + pp);
                    else
                        val_s[i] = 0.0f;
                }
            }
        } else {
            for (int i = tid; i < tb * NP; i += 128) {
                int tt = i / NP, nn = i - tt * NP;
                float kv = 0.0f, qv = 0.0f;
                if (nn < N) {
                    const float *row = src + (size_t)(c0 + tt) * in.ld + nn;
                    kv = add_partials(0.0f, row + kcol, in.S, in.stride);
                    if (in.silu)
                        kv = silu_f(kv);
                    if (MODE != 1) {
                        qv = add_partials(0.0f, row + qcol, in.S, in.stride);
                        if (in.silu)
                            qv = silu_f(qv);
                    }
                }
                key_s[i] = kv;
                if (MODE != 1)
                    qry_s[i] = qv;
            }
            for (int i = tid; i < tb * PT; i += 128) {
                int tt = i / PT, pp = i - tt * PT;
                float v = 0.0f;
                if (blockIdx.x * PT + pp < P) {
                    v = add_partials(0.0f, src + (size_t)(c0 + tt) * in.ld + vcol + pp, in.S, in.stride);
                    if (in.silu)
                        v = silu_f(v);
                }
                val_s[i] = v;
            }
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
        if (direct)
            copy_async_wait();
        __syncthreads();
        if (MODE == 1) {
            // The piece's own end state needs no row's state in between: over the batch's rows
            // S <- (product of their decays) S + sum_s (b_s times the decays after s) k_s v_s^T,
            // the rows taken last to first so that the decays after a row are a running product.
            // One multiply-add a value and row instead of a multiply and a multiply-add.
            float all = 1.0f;
            for (int tt = 0; tt < tb; tt++)
                all *= a_s[tt];
            run *= all;
#pragma unroll
            for (int i = 0; i < NR; i++)
                s[i] *= all;
            float after = 1.0f;
            for (int tt = tb - 1; tt >= 0; tt--) {
                float wv = b_s[tt] * after * val_s[tt * PT + pl];
                after *= a_s[tt];
                const float4 *kk = reinterpret_cast<const float4 *>(key_s + tt * NP) + ns;
#pragma unroll
                for (int i4 = 0; i4 < NR / 4; i4++)
                    if (i4 < cnt4) {
                        float4 k4 = kk[i4 * nsplit];
                        s[4 * i4 + 0] = fmaf(wv, k4.x, s[4 * i4 + 0]);
                        s[4 * i4 + 1] = fmaf(wv, k4.y, s[4 * i4 + 1]);
                        s[4 * i4 + 2] = fmaf(wv, k4.z, s[4 * i4 + 2]);
                        s[4 * i4 + 3] = fmaf(wv, k4.w, s[4 * i4 + 3]);
                    }
            }
        } else
        for (int tt = 0; tt < tb; tt++) {
            float a = a_s[tt], v = val_s[tt * PT + pl], bv = b_s[tt] * v;
            const float4 *kk = reinterpret_cast<const float4 *>(key_s + tt * NP) + ns;
            const float4 *qq = reinterpret_cast<const float4 *>(qry_s + tt * NP) + ns;
            float4 ac = make_float4(0.0f, 0.0f, 0.0f, 0.0f);     // four chains, added at the end
            run *= a;
#pragma unroll
            for (int i4 = 0; i4 < NR / 4; i4++)
                if (i4 < cnt4) {
                    float4 k4 = kk[i4 * nsplit];
                    s[4 * i4 + 0] = fmaf(bv, k4.x, a * s[4 * i4 + 0]);
                    s[4 * i4 + 1] = fmaf(bv, k4.y, a * s[4 * i4 + 1]);
                    s[4 * i4 + 2] = fmaf(bv, k4.z, a * s[4 * i4 + 2]);
                    s[4 * i4 + 3] = fmaf(bv, k4.w, a * s[4 * i4 + 3]);
                    if (MODE != 1) {
                        float4 q4 = qq[i4 * nsplit];
                        ac.x = fmaf(s[4 * i4 + 0], q4.x, ac.x);
                        ac.y = fmaf(s[4 * i4 + 1], q4.y, ac.y);
                        ac.z = fmaf(s[4 * i4 + 2], q4.z, ac.z);
                        ac.w = fmaf(s[4 * i4 + 3], q4.w, ac.w);
                    }
                }
            if (MODE != 1) {
                float acc = (ac.x + ac.y) + (ac.z + ac.w);
                for (int o = 16; o >= PW; o >>= 1)
                    acc += __shfl_xor_sync(0xffffffffu, acc, o);
                if (ns == 0 && live)
                    y[(size_t)(c0 + tt) * H * P + (size_t)h * P + p] = fmaf(dskip, v, acc);
            }
        }
    }
    // MODE 2: a sequence's last piece has walked the state to its end in the order of the one-pass
    // form; that is what the slot keeps (the carry pass's own end state differs from it in rounding)
    if (MODE == 2)
        st = state + (size_t)seq_slot[seq] * slot_stride + (size_t)h * N * P;
    if ((MODE != 2 || last_piece) && live) {
#pragma unroll
        for (int i = 0; i < NR; i++) {
            int nn = ((i >> 2) * nsplit + ns) * 4 + (i & 3);
            if (nn < N)
                st[(size_t)nn * P + p] = s[i];
        }
    }
    if (MODE == 1 && blockIdx.x == 0 && tid == 0)
        decays[(size_t)blockIdx.z * H + h] = run;
}

// Between the two passes over pieces: every sequence's state walks through its pieces,
// S <- decays[z] S + local[z], and local[z] is left holding the state its piece starts from
// (the state after the last piece is written by the second pass).  One thread per state value.
__global__ void __launch_bounds__(256)
matrix_state_carry_kernel(float *__restrict__ state, size_t slot_stride, const int32_t *__restrict__ row_seq,
                          const int32_t *__restrict__ seq_slot, float *__restrict__ local,
                          const float *__restrict__ decays, int n, int H, size_t per_head, int piece, int pieces)
{
    pdl_trigger();
    int seq = blockIdx.y;
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)H * per_head)
        return;
    int h = (int)(idx / per_head);
    int rows = first_row_of(row_seq, n, seq + 1) - first_row_of(row_seq, n, seq);
    if (rows <= 0)
        return;
    int used = rows >= 2 * piece ? (rows + piece - 1) / piece : 1;
    float *st = state + (size_t)seq_slot[seq] * slot_stride + idx;
    pdl_wait();
    float S = *st;
    // eight pieces' values are fetched together, then walked through in order
    for (int c0 = 0; c0 < used; c0 += 8) {
        float own[8], dec[8];
#pragma unroll
        for (int u = 0; u < 8; u++) {
            size_t z = (size_t)seq * pieces + min(c0 + u, used - 1);
            own[u] = local[z * H * per_head + idx];
            dec[u] = decays[z * H + h];
        }
#pragma unroll
        for (int u = 0; u < 8; u++)
            if (c0 + u < used) {
                size_t z = (size_t)seq * pieces + c0 + u;
                local[z * H * per_head + idx] = S;
                S = fmaf(dec[u], S, own[u]);
            }
    }
    (void)S;         // the slot's state is written by the second pass's last piece
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
                       int width, int parts, int keep)
{
    extern __shared__ float held[];          // the part's gated values, where they fit (keep != 0)
    __shared__ float red[32];
    pdl_trigger();
    int r = blockIdx.x, part = blockIdx.y, len = width / parts, c0 = part * len;
    pdl_wait();
    float ss = 0.0f;
    for (int c = c0 + threadIdx.x; c < c0 + len; c += blockDim.x) {
        float v = y[(size_t)r * width + c];
        if (pre != nullptr)
            v *= silu_f(add_partials(0.0f, pre + (size_t)r * pre_ld + pre_col0 + c, pre_S, pre_stride));
        if (keep)
            held[c - c0] = v;
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    float scale = 1.0f / sqrtf(ss / (float)len + eps);
    for (int c = c0 + threadIdx.x; c < c0 + len; c += blockDim.x) {
        float v;
        if (keep) {
            v = held[c - c0];
        } else {
            v = y[(size_t)r * width + c];
            if (pre != nullptr)
                v *= silu_f(add_partials(0.0f, pre + (size_t)r * pre_ld + pre_col0 + c, pre_S, pre_stride));
        }
        v = (v * scale) * w[c];
        if (post != nullptr)
            v *= sigmoid_f(add_partials(0.0f, post + (size_t)r * post_ld + post_col0 + c, post_S, post_stride));
        out[(size_t)r * width + c] = from_f<TO>(v);
    }
}

// The same for few rows: a cluster of C CTAs per (row, part), each with `cols` columns of the part
// held in shared memory; the CTAs exchange their sums of squares through one another's shared memory.
template <typename TO, int C>
__global__ void __launch_bounds__(256)
gated_part_norm_cluster_kernel(const float *__restrict__ y, const float *__restrict__ pre, int pre_S,
                               size_t pre_stride, int pre_ld, int pre_col0, const float *__restrict__ post,
                               int post_S, size_t post_stride, int post_ld, int post_col0,
                               const float *__restrict__ w, float eps, TO *__restrict__ out, int width, int parts,
                               int cols)
{
    extern __shared__ float held[];
    __shared__ float red[32];
    __shared__ float part_sq[C];
    pdl_trigger();
    uint32_t rank = cluster_rank();
    int idx = blockIdx.x / C, r = idx / parts, part = idx - r * parts, len = width / parts;
    int c0 = part * len + (int)rank * cols, c1 = min(part * len + len, c0 + cols);
    pdl_wait();
    float ss = 0.0f;
    for (int c = c0 + threadIdx.x; c < c1; c += blockDim.x) {
        float v = y[(size_t)r * width + c];
        if (pre != nullptr)
            v *= silu_f(add_partials(0.0f, pre + (size_t)r * pre_ld + pre_col0 + c, pre_S, pre_stride));
        held[c - c0] = v;
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    if (threadIdx.x < C)
        cluster_write(&part_sq[rank], threadIdx.x, ss);
    cluster_arrive();
    cluster_wait();
    float tot = 0.0f;
#pragma unroll
    for (int k = 0; k < C; k++)
        tot += part_sq[k];
    float scale = 1.0f / sqrtf(tot / (float)len + eps);
    for (int c = c0 + threadIdx.x; c < c1; c += blockDim.x) {
        float v = (held[c - c0] * scale) * w[c];
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

// The same for few rows: a cluster of C CTAs per row, each with `cols` columns of it held in
// shared memory; the CTAs exchange their sums of squares through one another's shared memory.
template <int C>
__global__ void __launch_bounds__(256)
pair_combine_cluster_kernel(const float *__restrict__ L, int SL, size_t strideL, const float *__restrict__ R, int SR,
                            size_t strideR, const float *__restrict__ wl, const float *__restrict__ wr, float sl,
                            float sr, float eps, float *__restrict__ out, int m, int cols)
{
    extern __shared__ float both[];          // [2, cols]
    __shared__ float red[32];
    __shared__ float part_l[C], part_r[C];
    pdl_trigger();
    uint32_t rank = cluster_rank();
    int r = blockIdx.x / C;
    int c0 = (int)rank * cols, c1 = min(m, c0 + cols);
    pdl_wait();
    float a = 0.0f, b = 0.0f;
    for (int c = c0 + threadIdx.x; c < c1; c += blockDim.x) {
        float u = add_partials(0.0f, L + (size_t)r * m + c, SL, strideL);
        float v = add_partials(0.0f, R + (size_t)r * m + c, SR, strideR);
        both[c - c0] = u;
        both[cols + c - c0] = v;
        a = fmaf(u, u, a);
        b = fmaf(v, v, b);
    }
    float fl = sl, fr = sr;
    if (wl != nullptr) {
        a = block_sum(a, red);
        b = block_sum(b, red);
        if (threadIdx.x < C) {
            cluster_write(&part_l[rank], threadIdx.x, a);
            cluster_write(&part_r[rank], threadIdx.x, b);
        }
        cluster_arrive();
        cluster_wait();
        float ta = 0.0f, tb = 0.0f;
#pragma unroll
        for (int k = 0; k < C; k++) {
            ta += part_l[k];
            tb += part_r[k];
        }
        fl = 1.0f / sqrtf(ta / (float)m + eps);
        fr = 1.0f / sqrtf(tb / (float)m + eps);
    } else {
        __syncthreads();
    }
    for (int c = c0 + threadIdx.x; c < c1; c += blockDim.x) {
        float u = both[c - c0], v = both[cols + c - c0];
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

// Into how many lanes a column of the state is split: the fewest that leave at most per_lane
// state values to a lane, more while a block's 128 / nsplit columns are more than twice P.
static int scan_nsplit(int N, int P, int per_lane)
{
    int ns = 1;
    while (ns < 32 && ((N + 4 * ns - 1) / (4 * ns)) * 4 > per_lane)
        ns *= 2;
    while (ns < 32 && 128 / ns >= 2 * P)
        ns *= 2;
    return ns;
}

// rows to a piece when long sequences are cut into pieces that run side by side
extern "C" int jb_matrix_state_piece(void) { return 128; }
// Floats of scratch for a step whose longest sequence brings max_len rows (0: one pass does it).
extern "C" long long jb_matrix_state_scratch(int n_seqs, int max_len, int H, int N, int P)
{
    int piece = jb_matrix_state_piece();
    if (max_len < 2 * piece)
        return 0;
    long long pieces = (max_len + piece - 1) / piece;
    long long need = (long long)n_seqs * pieces * ((long long)H * N * P + H);
    return need > (1ll << 28) ? 0 : need;       // more than 1 GiB of scratch: one pass after all
}

// src: float32 [S, n, ld] holding v (H P columns from val_col0), k and q (G N columns each);
// with dt (sums [dt_S, n, dt_ld], H columns from dt_col0) the selective form, otherwise
// decay [H].  state: [H, N, P] per slot.  y: float32 [n, H P].  scratch (with max_len, the most
// rows a sequence brings): jb_matrix_state_scratch floats, or null for one pass.
extern "C" int jb_matrix_state_scan(const float *src, int S, long long stride, int ld, int val_col0, int key_col0,
                                    int qry_col0, int silu, const float *dt, int dt_S, long long dt_stride,
                                    int dt_ld, int dt_col0, const float *dt_bias, const float *a_log,
                                    const float *skip, const float *decay, float *state, long long slot_stride,
                                    const int32_t *row_seq, const int32_t *seq_slot, float *y, int n, int n_seqs,
                                    int H, int G, int N, int P, int every_row_starts, float *scratch, int max_len,
                                    cudaStream_t st)
{
    if (n <= 0 || n_seqs <= 0)
        return JB_OK;
    if (H <= 0 || G <= 0 || H % G || N <= 0 || N > 1024 || P <= 0 || S <= 0 || src == nullptr || state == nullptr ||
        y == nullptr || (dt != nullptr && (dt_bias == nullptr || a_log == nullptr || dt_S <= 0)) ||
        (dt == nullptr && decay == nullptr) || H > 65535 || n_seqs > 65535 ||
        ld < val_col0 + H * P || ld < key_col0 + G * N || ld < qry_col0 + G * N)
        return JB_EINVAL;
    // 16 state values to a lane (more blocks, fewer registers, a shorter chain per row) where 32
    // lanes to a column are enough for that; 32 otherwise
    // (a decode step's one row per sequence moves the state and little else: fewer lanes to a
    // column then, so that a warp reads 32 bytes of a state row at a time)
    bool small = N <= 16 * 32 && !every_row_starts;
    int nsplit = scan_nsplit(N, P, small ? 16 : 32);
    if (((N + 4 * nsplit - 1) / (4 * nsplit)) * 4 > 32)
        return JB_EINVAL;
    constexpr int TB = 16;
    int PT = 128 / nsplit;
    int NP = (N + 4 * nsplit - 1) / (4 * nsplit) * (4 * nsplit);
    ScanIn in{src, S, (size_t)stride, ld, val_col0, key_col0, qry_col0, silu, dt, dt_S, (size_t)dt_stride, dt_ld,
              dt_col0, dt_bias, a_log, skip, decay};
    unsigned ptiles = (unsigned)((P + PT - 1) / PT);
    size_t smem = (size_t)TB * (2 * NP + PT + 2) * 4;
    int piece = jb_matrix_state_piece();
    bool whole = scratch == nullptr || every_row_starts || jb_matrix_state_scratch(n_seqs, max_len, H, N, P) == 0;
    int pieces = whole ? 1 : (max_len + piece - 1) / piece;
    if ((long long)n_seqs * pieces > 65535)
        return JB_EINVAL;
    size_t per_head = (size_t)N * P;
    float *local = scratch, *decays = whole ? nullptr : scratch + (size_t)n_seqs * pieces * H * per_head;
    dim3 grid(ptiles, (unsigned)H, (unsigned)(n_seqs * pieces));
#define JB_SCAN_N(NRV, MODE, NSV, SMEM)                                                                        \
    do {                                                                                                       \
        if ((SMEM) > 48 * 1024) {                                                                              \
            /* long states: the rows in shared memory need more than a kernel gets unasked */                  \
            static const bool asked = cudaFuncSetAttribute(matrix_state_scan_kernel<NRV, TB, MODE, NSV>,       \
                                                           cudaFuncAttributeMaxDynamicSharedMemorySize,        \
                                                           160 * 1024) == cudaSuccess;                         \
            (void)asked;                                                                                       \
        }                                                                                                      \
        launch(matrix_state_scan_kernel<NRV, TB, MODE, NSV>, grid, 128, (SMEM), st, in, state,                 \
               (size_t)slot_stride, row_seq, seq_slot, y, local, decays, n, H, G, N, P, nsplit,                \
               whole ? every_row_starts : 0, whole ? 0 : piece, pieces);                                       \
    } while (0)
    // the commonest shapes have kernels of their own: 128 or 64 state rows, 16 to a lane (prompts),
    // 128 rows, 32 to a lane (decode rows)
#define JB_SCAN(MODE, SMEM)                                              \
    do {                                                                 \
        if (small && nsplit == 8 && N == 128) JB_SCAN_N(16, MODE, 8, SMEM); \
        else if (small && nsplit == 4 && N == 64) JB_SCAN_N(16, MODE, 4, SMEM); \
        else if (!small && nsplit == 4 && N == 128) JB_SCAN_N(32, MODE, 4, SMEM); \
        else if (small) JB_SCAN_N(16, MODE, 0, SMEM);                    \
        else JB_SCAN_N(32, MODE, 0, SMEM);                               \
    } while (0)
    if (whole) {
        JB_SCAN(0, smem);
        return launch_status();
    }
    size_t smem1 = (size_t)TB * (NP + PT + 2) * 4;
    JB_SCAN(1, smem1);
    launch(matrix_state_carry_kernel, dim3((unsigned)(((size_t)H * per_head + 255) / 256), (unsigned)n_seqs), 256, 0, st,
           state, (size_t)slot_stride, row_seq, seq_slot, local, (const float *)decays, n, H, per_head, piece, pieces);
    JB_SCAN(2, smem);
#undef JB_SCAN
#undef JB_SCAN_N
    return launch_status();
}

extern "C" int jb_gated_part_norm(const float *y, const float *pre, int pre_S, long long pre_stride, int pre_ld,
                                  int pre_col0, const float *post, int post_S, long long post_stride, int post_ld,
                                  int post_col0, const float *w, float eps, void *out, int out_dt, int n, int width,
                                  int parts, int few_rows, cudaStream_t st)
{
    if (n <= 0)
        return JB_OK;
    if (width <= 0 || parts <= 0 || width % parts || parts > 65535 || y == nullptr || w == nullptr ||
        (pre != nullptr && (pre_S <= 0 || pre_ld < pre_col0 + width)) ||
        (post != nullptr && (post_S <= 0 || post_ld < post_col0 + width)))
        return JB_EINVAL;
    if (few_rows && n * parts <= 64 && width / parts >= 512 && out_dt == JB_BF16) {
        // few blocks otherwise: a cluster of CTAs per (row, part)
        constexpr int C = 4;
        int cols = (width / parts + C - 1) / C;
        if ((size_t)cols * 4 <= 40 * 1024) {
            launch_cluster(gated_part_norm_cluster_kernel<bf16, C>, dim3((unsigned)(n * parts * C)), 256, (size_t)cols * 4,
                           st, C, y, pre, pre_S, (size_t)pre_stride, pre_ld, pre_col0, post, post_S, (size_t)post_stride,
                           post_ld, post_col0, w, eps, (bf16 *)out, width, parts, cols);
            return launch_status();
        }
    }
    dim3 grid((unsigned)n, (unsigned)parts);
    size_t len = (size_t)(width / parts);
    int keep = len * 4 <= 40 * 1024 ? 1 : 0;
    size_t smem = keep ? len * 4 : 0;
    int threads = len >= 1024 ? 256 : 128;
    if (out_dt == JB_F32)
        launch(gated_part_norm_kernel<float>, grid, threads, smem, st, y, pre, pre_S, (size_t)pre_stride, pre_ld, pre_col0,
               post, post_S, (size_t)post_stride, post_ld, post_col0, w, eps, (float *)out, width, parts, keep);
    else if (out_dt == JB_BF16)
        launch(gated_part_norm_kernel<bf16>, grid, threads, smem, st, y, pre, pre_S, (size_t)pre_stride, pre_ld, pre_col0,
               post, post_S, (size_t)post_stride, post_ld, post_col0, w, eps, (bf16 *)out, width, parts, keep);
    else
        return JB_EINVAL;
    return launch_status();
}

extern "C" int jb_pair_combine(const float *L, int SL, long long strideL, const float *R, int SR, long long strideR,
                               const float *wl, const float *wr, float sl, float sr, float eps, float *out, int n,
                               int m, int few_rows, cudaStream_t st)
{
    if (n <= 0)
        return JB_OK;
    if (m <= 0 || SL <= 0 || SR <= 0 || L == nullptr || R == nullptr || out == nullptr || (wl == nullptr) != (wr == nullptr))
        return JB_EINVAL;
    if (few_rows && n <= 32 && m >= 512) {
        constexpr int C = 8;
        int cols = (m + C - 1) / C;
        if ((size_t)cols * 8 <= 40 * 1024) {
            launch_cluster(pair_combine_cluster_kernel<C>, dim3((unsigned)n * C), 256, (size_t)cols * 8, st, C, L, SL,
                           (size_t)strideL, R, SR, (size_t)strideR, wl, wr, sl, sr, eps, out, m, cols);
            return launch_status();
        }
    }
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

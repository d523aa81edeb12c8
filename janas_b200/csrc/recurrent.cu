// Recurrences along a sequence whose state is of fixed size: a short causal
// convolution over time on every channel of the residual stream, and the minGRU's
// gated running value.  The state lives per slot in float32 and is carried from
// step to step; everything here is computed in float32.
//
// Rows are the sequences' tokens one sequence after the other; row r belongs to
// sequence row_seq[r] of the step (slot seq_slot[row_seq[r]]) and stands at position
// row_pos[r].  The rows of one sequence are consecutive, so "the row k before r is of
// the same sequence" is row_seq[r - k] == row_seq[r].
#include "common.cuh"
#include "kernels.h"

namespace jb {

// ------------------------------------------------------------ short convolution
//
//   h_t = x_t + sum_{j < taps} w[:, j] * x_{t - taps + 1 + j}        (zeros before position 0)
//
// x: float32 [n, dm]; w: float32 [dm, taps].  state: float32 [taps - 1, dm] per slot,
// slot_stride floats from one slot's to the next's: the
// input at position p of a slot's sequence lies in row p % (taps - 1) until a later
// position takes the row.  Inputs of earlier steps are read from there, inputs of this
// step from x.  what & 1: h is written; what & 2: the rows that are among the last
// taps - 1 of their sequence in this step write their input into the state.  Both at
// once only where no row reads a state row that another row of the step writes: every
// sequence starts at position 0 (nothing is read) or brings one row (a thread reads
// before it writes its own).
template <typename TO, int V>
__global__ void __launch_bounds__(256)
short_conv_kernel(const float *__restrict__ x, const float *__restrict__ w, float *__restrict__ state,
                  size_t slot_stride, const int32_t *__restrict__ row_pos, const int32_t *__restrict__ row_seq,
                  const int32_t *__restrict__ seq_slot, TO *__restrict__ out, int n, int dm, int taps,
                  int what)
{
    pdl_trigger();
    int per_row = dm / V;
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n * per_row)
        return;
    int r = (int)(idx / per_row), c = (int)(idx - (size_t)r * per_row) * V;
    int pos = row_pos[r], seq = row_seq[r];
    int slot = seq_slot[seq];
    int keep = taps - 1;
    pdl_wait();
    float cur[V];
#pragma unroll
    for (int v = 0; v < V; v++)
        cur[v] = x[(size_t)r * dm + c + v];
    float *st = state != nullptr ? state + (size_t)slot * slot_stride : nullptr;
    if (what & 1) {
        float acc[V];
#pragma unroll
        for (int v = 0; v < V; v++)
            acc[v] = fmaf(w[(size_t)(c + v) * taps + taps - 1], cur[v], cur[v]);
        for (int k = 1; k <= keep; k++) {
            int p = pos - k;
            if (p < 0)
                break;
            const float *src = r - k >= 0 && row_seq[r - k] == seq ? x + (size_t)(r - k) * dm
                                                                  : st + (size_t)(p % keep) * dm;
#pragma unroll
            for (int v = 0; v < V; v++)
                acc[v] = fmaf(w[(size_t)(c + v) * taps + taps - 1 - k], src[c + v], acc[v]);
        }
#pragma unroll
        for (int v = 0; v < V; v++)
            out[(size_t)r * dm + c + v] = from_f<TO>(acc[v]);
    }
    if ((what & 2) && keep > 0 && (r + keep >= n || row_seq[r + keep] != seq)) {
#pragma unroll
        for (int v = 0; v < V; v++)
            st[(size_t)(pos % keep) * dm + c + v] = cur[v];
    }
}

// The same for 2 to 4 taps and a multiple of four channels, with x, the state and out on
// 16-byte boundaries: a thread has four channels of RB consecutive rows.  It keeps the last
// taps - 1 inputs in registers and moves along the rows, so that a row of x is read once
// (and the ones before a thread's first row once more); where a row starts a sequence's part
// of the step the inputs before it come from the state (or are zero before position 0).
template <typename TO, int TAPS, int RB>
__global__ void __launch_bounds__(256)
short_conv_rows_kernel(const float *__restrict__ x, const float *__restrict__ w, float *__restrict__ state,
                       size_t slot_stride, const int32_t *__restrict__ row_pos,
                       const int32_t *__restrict__ row_seq, const int32_t *__restrict__ seq_slot,
                       TO *__restrict__ out, int n, int dm, int what)
{
    constexpr int KEEP = TAPS - 1;
    pdl_trigger();
    int per_row = dm / 4;
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    int rb = (int)(idx / per_row), c = (int)(idx - (size_t)rb * per_row) * 4;
    int r0 = rb * RB, r1 = min(n, r0 + RB);
    if (r0 >= n)
        return;
    // wt[j]: tap j of the thread's four channels
    float4 wt[TAPS];
#pragma unroll
    for (int j = 0; j < TAPS; j++)
        wt[j] = make_float4(w[(size_t)c * TAPS + j], w[(size_t)(c + 1) * TAPS + j],
                            w[(size_t)(c + 2) * TAPS + j], w[(size_t)(c + 3) * TAPS + j]);
    pdl_wait();
    float4 hist[KEEP];          // hist[k - 1]: the input k positions back
    int prev_seq = -1;
    // the thread's rows are fetched together, then worked through in order
    float4 in_rows[RB];
    int in_pos[RB], in_seq[RB];
#pragma unroll
    for (int u = 0; u < RB; u++) {
        int rr = min(r0 + u, r1 - 1);
        in_rows[u] = load4(x + (size_t)rr * dm + c);
        in_pos[u] = row_pos[rr];
        in_seq[u] = row_seq[rr];
    }
#pragma unroll
    for (int u = 0; u < RB; u++) {
        int r = r0 + u;
        if (r >= r1)
            break;
        int pos = in_pos[u], seq = in_seq[u];
        float *st = state + (size_t)seq_slot[seq] * slot_stride;
        if (r == r0 || seq != prev_seq) {
#pragma unroll
            for (int k = 1; k <= KEEP; k++) {
                int p = pos - k;
                if (p < 0)
                    hist[k - 1] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                else if (r - k >= 0 && row_seq[r - k] == seq)
                    hist[k - 1] = load4(x + (size_t)(r - k) * dm + c);
                else
                    hist[k - 1] = load4(st + (size_t)(p % KEEP) * dm + c);
            }
        }
        prev_seq = seq;
        float4 cur = in_rows[u];
        if (what & 1) {
            float4 acc;
            acc.x = fmaf(wt[KEEP].x, cur.x, cur.x);
            acc.y = fmaf(wt[KEEP].y, cur.y, cur.y);
            acc.z = fmaf(wt[KEEP].z, cur.z, cur.z);
            acc.w = fmaf(wt[KEEP].w, cur.w, cur.w);
#pragma unroll
            for (int k = 1; k <= KEEP; k++) {
                acc.x = fmaf(wt[KEEP - k].x, hist[k - 1].x, acc.x);
                acc.y = fmaf(wt[KEEP - k].y, hist[k - 1].y, acc.y);
                acc.z = fmaf(wt[KEEP - k].z, hist[k - 1].z, acc.z);
                acc.w = fmaf(wt[KEEP - k].w, hist[k - 1].w, acc.w);
            }
            store4(out + (size_t)r * dm + c, acc);
        }
        if ((what & 2) && (r + KEEP >= n || row_seq[r + KEEP] != seq))
            store4(st + (size_t)(pos % KEEP) * dm + c, cur);
#pragma unroll
        for (int k = KEEP - 1; k > 0; k--)
            hist[k] = hist[k - 1];
        hist[0] = cur;
    }
}

// A causal convolution over time on C columns of a product's sums, without the input
// added:  out[r, c] = act(bias[c] + sum_{j < taps} w[c, j] * u_{t - taps + 1 + j}[c]),
// u = the sums in columns col0 .. col0 + C - 1 of [S, n, ld]; zeros before position 0.
// State, `what` and the rule for one launch or two are short_conv_kernel's: a ring of the
// last taps - 1 inputs per slot, [taps - 1, C].  act 1: silu.  out: [n, out_ld] with the
// result in its first C columns.  One thread per (row, column).
template <typename TO>
__global__ void __launch_bounds__(256)
causal_conv_kernel(const float *__restrict__ u, int S, size_t stride, int ld, int col0,
                   const float *__restrict__ w, const float *__restrict__ bias, float *__restrict__ state,
                   size_t slot_stride, const int32_t *__restrict__ row_pos, const int32_t *__restrict__ row_seq,
                   const int32_t *__restrict__ seq_slot, TO *__restrict__ out, int out_ld, int n, int C, int taps,
                   int act, int what)
{
    pdl_trigger();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n * C)
        return;
    int r = (int)(idx / C), c = (int)(idx - (size_t)r * C);
    int pos = row_pos[r], seq = row_seq[r];
    int keep = taps - 1;
    float *st = state != nullptr ? state + (size_t)seq_slot[seq] * slot_stride : nullptr;
    pdl_wait();
    float cur = add_partials(0.0f, u + (size_t)r * ld + col0 + c, S, stride);
    if (what & 1) {
        float acc = bias != nullptr ? bias[c] : 0.0f;
        acc = fmaf(w[(size_t)c * taps + taps - 1], cur, acc);
        for (int k = 1; k <= keep; k++) {
            int p = pos - k;
            if (p < 0)
                break;
            float v = r - k >= 0 && row_seq[r - k] == seq
                          ? add_partials(0.0f, u + (size_t)(r - k) * ld + col0 + c, S, stride)
                          : st[(size_t)(p % keep) * C + c];
            acc = fmaf(w[(size_t)c * taps + taps - 1 - k], v, acc);
        }
        if (act == 1)
            acc = acc / (1.0f + expf(-acc));
        out[(size_t)r * out_ld + c] = from_f<TO>(acc);
    }
    if ((what & 2) && keep > 0 && (r + keep >= n || row_seq[r + keep] != seq))
        st[(size_t)(pos % keep) * C + c] = cur;
}

// The same for one sum (S = 1), 2 to 4 taps and a multiple of four columns, with everything on
// 16-byte boundaries: a thread has four columns of RB consecutive rows, keeps the last taps - 1
// inputs in registers and moves along the rows (as short_conv_rows_kernel does).  The sums run
// in the order of causal_conv_kernel, so a row's bits are the same on either way.
template <typename TO, int TAPS, int RB>
__global__ void __launch_bounds__(256)
causal_conv_rows_kernel(const float *__restrict__ u, int ld, int col0, const float *__restrict__ w,
                        const float *__restrict__ bias, float *__restrict__ state, size_t slot_stride,
                        const int32_t *__restrict__ row_pos, const int32_t *__restrict__ row_seq,
                        const int32_t *__restrict__ seq_slot, TO *__restrict__ out, int out_ld, int n, int C,
                        int act, int what)
{
    constexpr int KEEP = TAPS - 1;
    pdl_trigger();
    int per_row = C / 4;
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    int rb = (int)(idx / per_row), c = (int)(idx - (size_t)rb * per_row) * 4;
    int r0 = rb * RB, r1 = min(n, r0 + RB);
    if (r0 >= n)
        return;
    float4 wt[TAPS];
#pragma unroll
    for (int j = 0; j < TAPS; j++)
        wt[j] = make_float4(w[(size_t)c * TAPS + j], w[(size_t)(c + 1) * TAPS + j], w[(size_t)(c + 2) * TAPS + j],
                            w[(size_t)(c + 3) * TAPS + j]);
    float4 bs = bias != nullptr ? load4(bias + c) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    pdl_wait();
    const float *in = u + col0 + c;
    float4 hist[KEEP];          // hist[k - 1]: the input k positions back
    int prev_seq = -1;
    float4 in_rows[RB];
    int in_pos[RB], in_seq[RB];
#pragma unroll
    for (int q = 0; q < RB; q++) {
        int rr = min(r0 + q, r1 - 1);
        in_rows[q] = load4(in + (size_t)rr * ld);
        in_pos[q] = row_pos[rr];
        in_seq[q] = row_seq[rr];
    }
#pragma unroll
    for (int q = 0; q < RB; q++) {
        int r = r0 + q;
        if (r >= r1)
            break;
        int pos = in_pos[q], seq = in_seq[q];
        float *st = state + (size_t)seq_slot[seq] * slot_stride;
        if (r == r0 || seq != prev_seq) {
#pragma unroll
            for (int k = 1; k <= KEEP; k++) {
                int p = pos - k;
                if (p < 0)
                    hist[k - 1] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                else if (r - k >= 0 && row_seq[r - k] == seq)
                    hist[k - 1] = load4(in + (size_t)(r - k) * ld);
                else
                    hist[k - 1] = load4(st + (size_t)(p % KEEP) * C + c);
            }
        }
        prev_seq = seq;
        float4 cur = in_rows[q];
        if (what & 1) {
            float4 acc = bs;
            acc.x = fmaf(wt[KEEP].x, cur.x, acc.x);
            acc.y = fmaf(wt[KEEP].y, cur.y, acc.y);
            acc.z = fmaf(wt[KEEP].z, cur.z, acc.z);
            acc.w = fmaf(wt[KEEP].w, cur.w, acc.w);
#pragma unroll
            for (int k = 1; k <= KEEP; k++) {
                if (pos - k < 0)
                    break;
                acc.x = fmaf(wt[KEEP - k].x, hist[k - 1].x, acc.x);
                acc.y = fmaf(wt[KEEP - k].y, hist[k - 1].y, acc.y);
                acc.z = fmaf(wt[KEEP - k].z, hist[k - 1].z, acc.z);
                acc.w = fmaf(wt[KEEP - k].w, hist[k - 1].w, acc.w);
            }
            if (act == 1) {
                acc.x = acc.x / (1.0f + expf(-acc.x));
                acc.y = acc.y / (1.0f + expf(-acc.y));
                acc.z = acc.z / (1.0f + expf(-acc.z));
                acc.w = acc.w / (1.0f + expf(-acc.w));
            }
            store4<TO>(out + (size_t)r * out_ld + c, acc);
        }
        if ((what & 2) && (r + KEEP >= n || row_seq[r + KEEP] != seq))
            *reinterpret_cast<float4 *>(st + (size_t)(pos % KEEP) * C + c) = cur;
#pragma unroll
        for (int k = KEEP - 1; k >= 1; k--)
            hist[k] = hist[k - 1];
        hist[0] = cur;
    }
}

// ---------------------------------------------------------------------- minGRU
//
//   z = sigmoid(P_z + b_z);  u = P_x + b_x;  c = u + 1/2 (u >= 0), sigmoid(u) (u < 0)
//   S_t = (1 - z_t) S_{t-1} + z_t c_t;   out_t = S_t * silu(P_g)
//
// P: the sums [S, n, ld] of one product over the mixer's input whose columns are
// [z | x | g] from col0 on, W each; bias: float32 [3 W] over those columns or null.
// state: float32 [slots, W], a sequence's S after its last computed token.
struct GruIn {
    const float *P;
    int S;
    size_t stride;
    int ld, col0;
    const float *bias;
    int W;
};

// FAST: the hardware's approximate exponential and division (the bfloat16 path, whose
// results are rounded to 8 bits of mantissa afterwards); otherwise expf and a true division
template <bool FAST> __device__ __forceinline__ float sigmoidf_(float v)
{
    return FAST ? __fdividef(1.0f, 1.0f + __expf(-v)) : 1.0f / (1.0f + expf(-v));
}



// a_t = 1 - z_t, b_t = z_t c_t from the gates' sums (bias included)
template <bool FAST>
__device__ __forceinline__ void gru_coef(float zs, float u, float &a, float &b)
{
    float z = sigmoidf_<FAST>(zs);
    float c = u >= 0.0f ? u + 0.5f : sigmoidf_<FAST>(u);
    a = 1.0f - z;
    b = z * c;
}

// GRU_U: rows whose gates a thread of the minGRU kernels computes together (8 along a piece,
// 1 where every row is a piece of its own).
// The sums of column block `blk` (0 z, 1 x, 2 g) of channel ch for the GRU_U rows from rb on
// (rows past r1 - 1 repeat that row: nothing branches, so the loads go out together).
template <int GRU_U>
__device__ __forceinline__ void gru_sums(const GruIn &in, int blk, int rb, int r1, int ch, float *out)
{
    float bias = in.bias != nullptr ? in.bias[blk * in.W + ch] : 0.0f;
    const float *p = in.P + in.col0 + (size_t)blk * in.W + ch;
    if (in.S == 1) {
#pragma unroll
        for (int u = 0; u < GRU_U; u++)
            out[u] = p[(size_t)min(rb + u, r1 - 1) * in.ld];
#pragma unroll
        for (int u = 0; u < GRU_U; u++)
            out[u] += bias;
    } else {
#pragma unroll
        for (int u = 0; u < GRU_U; u++)
            out[u] = add_partials(bias, p + (size_t)min(rb + u, r1 - 1) * in.ld, in.S, in.stride);
    }
}

// Rows are cut into pieces of `piece` consecutive rows of the step; a thread owns one
// channel of one piece.  Over a piece the recurrence is S -> A S + B; the first row of a
// sequence within the step starts from the slot's state instead (A = 0).  This kernel
// leaves A and B of every piece in AB [pieces, 2, W] and a copy of the state each
// sequence starts from in init [sequences, W].
template <int GRU_U, bool FAST>
__global__ void __launch_bounds__(128)
mingru_pieces_kernel(GruIn in, const float *__restrict__ state, const int32_t *__restrict__ row_seq,
                     const int32_t *__restrict__ seq_slot, float *__restrict__ AB, float *__restrict__ init,
                     int n, int piece)
{
    pdl_trigger();
    int ch = blockIdx.x * blockDim.x + threadIdx.x, pc = blockIdx.y;
    if (ch >= in.W)
        return;
    pdl_wait();
    int r0 = pc * piece, r1 = min(n, r0 + piece);
    float A = 1.0f, B = 0.0f;
    // GRU_U rows at a time: their gates are fetched and computed together, so that the chain
    // through the rows is one of multiply-adds, not of memory latencies
    int before = r0 > 0 ? row_seq[r0 - 1] : -1;
    // the next rows' sums are asked for before this batch's chain is walked
    float nz[GRU_U], nu[GRU_U];
    int nsq[GRU_U];
    gru_sums<GRU_U>(in, 0, r0, r1, ch, nz);
    gru_sums<GRU_U>(in, 1, r0, r1, ch, nu);
#pragma unroll
    for (int u = 0; u < GRU_U; u++)
        nsq[u] = row_seq[min(r0 + u, r1 - 1)];
    for (int rb = r0; rb < r1; rb += GRU_U) {
        float a[GRU_U], b[GRU_U];
        int sq[GRU_U];
#pragma unroll
        for (int u = 0; u < GRU_U; u++) {
            gru_coef<FAST>(nz[u], nu[u], a[u], b[u]);
            sq[u] = nsq[u];
        }
        if (rb + GRU_U < r1) {
            gru_sums<GRU_U>(in, 0, rb + GRU_U, r1, ch, nz);
            gru_sums<GRU_U>(in, 1, rb + GRU_U, r1, ch, nu);
#pragma unroll
            for (int u = 0; u < GRU_U; u++)
                nsq[u] = row_seq[min(rb + GRU_U + u, r1 - 1)];
        }
#pragma unroll
        for (int u = 0; u < GRU_U; u++)
            if (rb + u < r1) {
                int seq = sq[u];
                if (seq != before) {
                    float s0 = state[(size_t)seq_slot[seq] * in.W + ch];
                    init[(size_t)seq * in.W + ch] = s0;
                    A = 0.0f;
                    B = fmaf(a[u], s0, b[u]);
                } else {
                    A *= a[u];
                    B = fmaf(a[u], B, b[u]);
                }
                before = seq;
            }
    }
    AB[((size_t)pc * 2) * in.W + ch] = A;
    AB[((size_t)pc * 2 + 1) * in.W + ch] = B;
}

// The value each piece starts from: carry [pieces, W], piece after piece.
__global__ void __launch_bounds__(128)
mingru_carry_kernel(const float *__restrict__ AB, float *__restrict__ carry, int W, int pieces)
{
    pdl_trigger();
    int ch = blockIdx.x * blockDim.x + threadIdx.x;
    if (ch >= W)
        return;
    pdl_wait();
    float s = 0.0f;
    for (int pc = 0; pc < pieces; pc++) {
        carry[(size_t)pc * W + ch] = s;
        s = fmaf(AB[((size_t)pc * 2) * W + ch], s, AB[((size_t)pc * 2 + 1) * W + ch]);
    }
}

// The recurrence itself over each piece, from the piece's carry (null: nothing is
// carried into a piece: one piece in all, or every row starts a sequence), with the
// output and the new state.  init null: a sequence's start is read from the state
// itself (only where the thread that reads it is the one that writes it: one piece, or
// one row per sequence).
template <typename TO, int GRU_U>
__global__ void __launch_bounds__(128)
mingru_scan_kernel(GruIn in, float *__restrict__ state, const int32_t *__restrict__ row_seq,
                   const int32_t *__restrict__ seq_slot, const float *__restrict__ carry,
                   const float *__restrict__ init, TO *__restrict__ out, int n, int piece)
{
    constexpr bool FAST = sizeof(TO) == 2;
    pdl_trigger();
    int ch = blockIdx.x * blockDim.x + threadIdx.x, pc = blockIdx.y;
    if (ch >= in.W)
        return;
    pdl_wait();
    int r0 = pc * piece, r1 = min(n, r0 + piece);
    float s = carry != nullptr ? carry[(size_t)pc * in.W + ch] : 0.0f;
    int before = r0 > 0 ? row_seq[r0 - 1] : -1;
    // the next rows' sums are asked for before this batch's chain is walked
    float nz[GRU_U], nu[GRU_U], ng[GRU_U];
    int nsq[GRU_U];
    gru_sums<GRU_U>(in, 0, r0, r1, ch, nz);
    gru_sums<GRU_U>(in, 1, r0, r1, ch, nu);
    gru_sums<GRU_U>(in, 2, r0, r1, ch, ng);
#pragma unroll
    for (int u = 0; u < GRU_U; u++)
        nsq[u] = row_seq[min(r0 + u, r1 - 1)];
    for (int rb = r0; rb < r1; rb += GRU_U) {
        float a[GRU_U], b[GRU_U], gs[GRU_U];
        int sq[GRU_U + 1];
#pragma unroll
        for (int u = 0; u < GRU_U; u++) {
            gru_coef<FAST>(nz[u], nu[u], a[u], b[u]);
            gs[u] = ng[u] * sigmoidf_<FAST>(ng[u]);
            sq[u] = nsq[u];
        }
        if (rb + GRU_U < r1) {
            gru_sums<GRU_U>(in, 0, rb + GRU_U, r1, ch, nz);
            gru_sums<GRU_U>(in, 1, rb + GRU_U, r1, ch, nu);
            gru_sums<GRU_U>(in, 2, rb + GRU_U, r1, ch, ng);
#pragma unroll
            for (int u = 0; u < GRU_U; u++)
                nsq[u] = row_seq[min(rb + GRU_U + u, r1 - 1)];
        }
        int last = min(GRU_U, r1 - rb);
        int after = rb + last < n ? row_seq[rb + last] : -1;
#pragma unroll
        for (int u = 0; u < GRU_U; u++)
            if (rb + u < r1) {
                int r = rb + u, seq = sq[u];
                if (seq != before)
                    s = init != nullptr ? init[(size_t)seq * in.W + ch] : state[(size_t)seq_slot[seq] * in.W + ch];
                s = fmaf(a[u], s, b[u]);
                out[(size_t)r * in.W + ch] = from_f<TO>(s * gs[u]);
                int next = u + 1 < last ? sq[u + 1 < GRU_U ? u + 1 : u] : after;
                if (next != seq)
                    state[(size_t)seq_slot[seq] * in.W + ch] = s;
                before = seq;
            }
    }
}

}  // namespace jb

using namespace jb;

// what: 1 = write h, 2 = write the state, 3 = both (see short_conv_kernel for when).
// state may be null with taps == 1.
extern "C" int jb_short_conv(const float *x, const float *w, float *state, long long slot_stride,
                             const int32_t *row_pos,
                             const int32_t *row_seq, const int32_t *seq_slot, void *out, int out_dt, int n,
                             int dm, int taps, int what, cudaStream_t st)
{
    if (n <= 0)
        return JB_OK;
    if (dm <= 0 || taps < 1 || (taps > 1 && (state == nullptr || slot_stride < (long long)(taps - 1) * dm)) || !(what & 3) ||
        ((what & 1) && out == nullptr))
        return JB_EINVAL;
    bool vec = dm % 4 == 0;
    auto al16 = [](const void *p) { return ((uintptr_t)p & 15) == 0; };
    if (vec && taps >= 2 && taps <= 4 && al16(x) && al16(state) && al16(out) && slot_stride % 4 == 0 &&
        (out_dt == JB_F32 || out_dt == JB_BF16)) {
        // many rows: eight to a thread; few: one (a decode step's rows are all of other sequences)
        bool many = (size_t)n * (dm / 4) >= (size_t)8 * 148 * 1024;
        int rbs = many ? 8 : 1;
        size_t threads = (size_t)((n + rbs - 1) / rbs) * (dm / 4);
        unsigned g = (unsigned)((threads + 255) / 256);
#define JB_SCR(TO, T, RB)                                                                             \
    launch(short_conv_rows_kernel<TO, T, RB>, g, 256, 0, st, x, w, state, (size_t)slot_stride, row_pos, \
           row_seq, seq_slot, (TO *)out, n, dm, what)
#define JB_SCR_T(TO, RB)                                                                              \
    do {                                                                                              \
        if (taps == 2) JB_SCR(TO, 2, RB);                                                             \
        else if (taps == 3) JB_SCR(TO, 3, RB);                                                        \
        else JB_SCR(TO, 4, RB);                                                                       \
    } while (0)
        if (out_dt == JB_F32) {
            if (many) JB_SCR_T(float, 8); else JB_SCR_T(float, 1);
        } else {
            if (many) JB_SCR_T(bf16, 8); else JB_SCR_T(bf16, 1);
        }
#undef JB_SCR_T
#undef JB_SCR
        return launch_status();
    }
    size_t total = (size_t)n * (vec ? dm / 4 : dm);
    unsigned grid = (unsigned)((total + 255) / 256);
#define JB_SC(TO, V)                                                                                  \
    launch(short_conv_kernel<TO, V>, grid, 256, 0, st, x, w, state, (size_t)slot_stride, row_pos, row_seq, seq_slot, (TO *)out, \
           n, dm, taps, what)
    if (out_dt == JB_F32) {
        if (vec) JB_SC(float, 4); else JB_SC(float, 1);
    } else if (out_dt == JB_BF16) {
        if (vec) JB_SC(bf16, 4); else JB_SC(bf16, 1);
    } else {
        return JB_EINVAL;
    }
#undef JB_SC
    return launch_status();
}

// u: float32 [S, n, ld]; w: float32 [C, taps]; bias: float32 [C] or null; state: float32
// [taps - 1, C] per slot (null with taps == 1).  out: [n, out_ld] in out_dt.
extern "C" int jb_causal_conv(const float *u, int S, long long stride, int ld, int col0, const float *w,
                              const float *bias, float *state, long long slot_stride, const int32_t *row_pos,
                              const int32_t *row_seq, const int32_t *seq_slot, void *out, int out_dt, int out_ld,
                              int n, int C, int taps, int act, int what, cudaStream_t st)
{
    if (n <= 0 || C <= 0 || !(what & 3))
        return JB_OK;
    if (taps < 1 || S <= 0 || ld < col0 + C || col0 < 0 || out_ld < C || u == nullptr || w == nullptr ||
        (taps > 1 && state == nullptr) || ((what & 1) && out == nullptr) || (act != 0 && act != 1))
        return JB_EINVAL;
    auto al16 = [](const void *p) { return ((uintptr_t)p & 15) == 0; };
    if (S == 1 && taps >= 2 && taps <= 4 && C % 4 == 0 && ld % 4 == 0 && col0 % 4 == 0 && out_ld % 4 == 0 &&
        slot_stride % 4 == 0 && al16(u) && al16(bias) && al16(state) && al16(out)) {
        // many rows: eight to a thread; few: one (a decode step's rows are all of other sequences)
        bool many = (size_t)n * (C / 4) >= (size_t)8 * 148 * 1024;
        int rbs = many ? 8 : 1;
        size_t threads = (size_t)((n + rbs - 1) / rbs) * (C / 4);
        unsigned g = (unsigned)((threads + 255) / 256);
#define JB_CCR(TO, T, RB)                                                                                  \
    launch(causal_conv_rows_kernel<TO, T, RB>, g, 256, 0, st, u, ld, col0, w, bias, state, (size_t)slot_stride, \
           row_pos, row_seq, seq_slot, (TO *)out, out_ld, n, C, act, what)
#define JB_CCR_T(TO, RB)                                                                                   \
    do {                                                                                                   \
        if (taps == 2) JB_CCR(TO, 2, RB);                                                                  \
        else if (taps == 3) JB_CCR(TO, 3, RB);                                                             \
        else JB_CCR(TO, 4, RB);                                                                            \
    } while (0)
        if (out_dt == JB_F32) {
            if (many) JB_CCR_T(float, 8); else JB_CCR_T(float, 1);
            return launch_status();
        }
        if (out_dt == JB_BF16) {
            if (many) JB_CCR_T(bf16, 8); else JB_CCR_T(bf16, 1);
            return launch_status();
        }
#undef JB_CCR_T
#undef JB_CCR
    }
    unsigned grid = (unsigned)(((size_t)n * C + 255) / 256);
    if (out_dt == JB_F32)
        launch(causal_conv_kernel<float>, grid, 256, 0, st, u, S, (size_t)stride, ld, col0, w, bias, state,
               (size_t)slot_stride, row_pos, row_seq, seq_slot, (float *)out, out_ld, n, C, taps, act, what);
    else if (out_dt == JB_BF16)
        launch(causal_conv_kernel<bf16>, grid, 256, 0, st, u, S, (size_t)stride, ld, col0, w, bias, state,
               (size_t)slot_stride, row_pos, row_seq, seq_slot, (bf16 *)out, out_ld, n, C, taps, act, what);
    else
        return JB_EINVAL;
    return launch_status();
}

// Floats of scratch for n rows cut into pieces (0 when one launch does it).
extern "C" int jb_mingru_piece(void) { return 64; }
extern "C" long long jb_mingru_scratch(int n, int n_seqs, int W, int every_row_starts)
{
    int piece = jb_mingru_piece();
    if (every_row_starts || n <= piece)
        return 0;
    long long pieces = (n + piece - 1) / piece;
    return pieces * 3 * W + (long long)n_seqs * W;
}

// P: float32 [S, n, ld]; the mixer's columns [z | x | g] start at col0.  out: [n, W] in
// out_dt.  every_row_starts: each row is the one new token of its sequence.
extern "C" int jb_mingru(const float *P, int S, long long stride, int ld, int col0, const float *bias,
                         float *state, const int32_t *row_seq, const int32_t *seq_slot, float *scratch,
                         void *out, int out_dt, int n, int n_seqs, int W, int every_row_starts,
                         cudaStream_t st)
{
    if (n <= 0)
        return JB_OK;
    if (W <= 0 || S <= 0 || ld < col0 + 3 * W || state == nullptr || (out_dt != JB_F32 && out_dt != JB_BF16))
        return JB_EINVAL;
    GruIn in{P, S, (size_t)stride, ld, col0, bias, W};
    int piece = every_row_starts ? 1 : jb_mingru_piece();
    int pieces = (n + piece - 1) / piece;
    dim3 grid((unsigned)((W + 127) / 128), (unsigned)pieces);
    const float *carry = nullptr, *init = nullptr;
    if (!every_row_starts && pieces > 1) {
        if (scratch == nullptr)
            return JB_EINVAL;
        float *AB = scratch, *cr = scratch + (size_t)pieces * 2 * W, *ini = cr + (size_t)pieces * W;
        if (out_dt == JB_BF16)
            launch(mingru_pieces_kernel<8, true>, grid, 128, 0, st, in, (const float *)state, row_seq, seq_slot,
                   AB, ini, n, piece);
        else
            launch(mingru_pieces_kernel<8, false>, grid, 128, 0, st, in, (const float *)state, row_seq, seq_slot,
                   AB, ini, n, piece);
        launch(mingru_carry_kernel, (unsigned)((W + 127) / 128), 128, 0, st, (const float *)AB, cr, W, pieces);
        carry = cr;
        init = ini;
    }
    if (out_dt == JB_F32 && piece == 1)
        launch(mingru_scan_kernel<float, 1>, grid, 128, 0, st, in, state, row_seq, seq_slot, carry, init,
               (float *)out, n, piece);
    else if (out_dt == JB_F32)
        launch(mingru_scan_kernel<float, 8>, grid, 128, 0, st, in, state, row_seq, seq_slot, carry, init,
               (float *)out, n, piece);
    else if (piece == 1)
        launch(mingru_scan_kernel<bf16, 1>, grid, 128, 0, st, in, state, row_seq, seq_slot, carry, init,
               (bf16 *)out, n, piece);
    else
        launch(mingru_scan_kernel<bf16, 8>, grid, 128, 0, st, in, state, row_seq, seq_slot, carry, init,
               (bf16 *)out, n, piece);
    return launch_status();
}

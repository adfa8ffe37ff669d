// The gated delta rule: a linear recurrence whose state decays by a gate computed from the token and is
// corrected towards the token's value along its key, over a float32 state per request and head.
//
//   x      = the rows of one stacked projection: q | k (n_qk heads of d each) | v (nh heads of dv), and one
//            logit a head for beta and for the decay
//   q, k, v = silu(conv(x)): a causal convolution over the request's tokens per channel, `taps` long, the last
//            tap on the current token, zeros before the request's start
//   q, k   = q / sqrt(sum(q^2) + unit_eps) * q_scale,  k / sqrt(sum(k^2) + unit_eps)        per head
//   beta   = sigmoid(x_b),   g = exp(-exp(A_log_h) * softplus(x_a + dt_bias_h))             per head
//   S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q                             per head, S [d, dv]
//
// (head h reads q and k of head h / (nh / n_qk)).  Everything after the projection is float32.
//
// A request's state slot holds S transposed ([nh, dv, d], a column's entries contiguous) followed by the last
// taps - 1 rows of x's q | k | v columns, [taps - 1, C] as float32 (exact for either element type); a request
// whose first token is in this step starts from zeros in both.
//
// prepare: one warp a (token, head of q, k or v), and one more a token for beta and the decay; writes float32 rows
//          [q | k | v | beta | ln g].  It reads the convolution's tail from the slot and leaves it as it is.
// scan:    (steps of single tokens and short portions) columns of S evolve independently: a CTA takes (request,
//          head, 16 columns), 16 threads share a column (each a contiguous share of its entries in registers) and
//          walk the request's tokens of this step in order; the column's dot product with k is summed over the 16
//          threads by shuffles, the read-out's partial sums after each tile of tokens.  The request's CTAs also
//          move the slot's convolution tail on, a share of the channels each (every reader of the old one is
//          done: the prepare kernel has finished).
// chunks:  (steps with prompts) the same CTAs and threads take 16 tokens at a time.  With L_t the sum of ln g
//          over the chunk's tokens up to t and S0 the state before the chunk,
//              u_t = beta_t (v_t - e^{L_t} S0^T k_t) - sum_{i<t} beta_t e^{L_t - L_i} (k_t . k_i) u_i
//              o_t = e^{L_t} S0^T q_t + sum_{i<=t} e^{L_t - L_i} (q_t . k_i) u_i
//              S   = e^{L_15} S0 + sum_t e^{L_15 - L_t} k_t u_t^T
//          which is the recurrence written out.  The products with S0 of all 16 tokens are independent (summed
//          over a column's 16 threads by a transposing butterfly, after which thread t of the column holds token
//          t's), the triangular system is solved by 16 broadcasts inside the column's half-warp, and the state
//          takes the 16 outer products at once: the chain from token to token shrinks from a shuffle reduction a
//          token to one broadcast and one multiply-add.  The dot products k_t . k_i and q_t . k_i of tokens in the
//          same chunk do not depend on S: a kernel before (gram: a warp a (token, q/k head)) leaves them by
//          (token, tokens back).  Every exponent is <= 0.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int MAX_D = 512;                       // head sizes of q and k up to 512 (16 entries a lane in prepare)
constexpr int MAX_TAPS = 8;
constexpr int PREP_WARPS = 4;

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

struct Seqs {
    const int* cu_seqlens;      // [B + 1] first row of every request among the step's tokens
    const int* ctx_lens;        // [B] tokens of the request once this step is done
    const int* state_slots;     // [B]
    const int* seq_of_token;    // [T]
};

// The input of channel c (of C) that lies `back` tokens before local index `li` of a request's portion that
// starts at row `row0`: from this step's rows, from the slot's tail, or zero before the request's start.
template <typename T>
__device__ __forceinline__ float conv_input(const T* __restrict__ x, long long stride, int row0, int src, int c, int C,
                                            const float* __restrict__ tail, int taps, bool fresh) {
    if (src >= 0) return to_f<T>(x[(size_t)(row0 + src) * stride + c]);
    return fresh ? 0.f : tail[(size_t)(taps - 1 + src) * C + c];
}

template <typename T>
__global__ __launch_bounds__(PREP_WARPS * 32) void delta_prepare_kernel(
    const T* __restrict__ proj, long long stride, int qkv_off, int b_off, int a_off,
    const float* __restrict__ conv_w, const float* __restrict__ a_log, const float* __restrict__ dt_bias,
    const float* __restrict__ state, long long state_stride, long long tail_off, Seqs sq,
    float* __restrict__ act, int n_units, int nh, int n_qk, int d, int dv, int taps, float unit_eps, float q_scale) {
    pdl_wait_and_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int unit = blockIdx.x * PREP_WARPS + warp;
    if (unit >= n_units) return;
    const int per = 2 * n_qk + nh + 1;
    const int t = unit / per, u = unit - t * per;
    const int C = 2 * n_qk * d + nh * dv;
    const int AW = C + 2 * nh;
    float* arow = act + (size_t)t * AW;
    if (u == per - 1) {
        const T* row = proj + (size_t)t * stride;
        for (int h = lane; h < nh; h += 32) {
            arow[C + h] = 1.0f / (1.0f + expf(-to_f<T>(row[b_off + h])));
            // ln g, kept finite so that differences of its sums are defined (e^x is 0 long before)
            arow[C + nh + h] = fmaxf(-expf(a_log[h]) * softplus_f(to_f<T>(row[a_off + h]) + dt_bias[h]), -1e30f);
        }
        return;
    }
    const int b = sq.seq_of_token[t];
    const int row0 = sq.cu_seqlens[b], n = sq.cu_seqlens[b + 1] - row0;
    const int li = t - row0;
    const bool fresh = sq.ctx_lens[b] - n == 0;
    const float* tail = state + (size_t)sq.state_slots[b] * state_stride + tail_off;
    const bool unit_norm = u < 2 * n_qk;
    const int width = unit_norm ? d : dv;
    const int c0 = unit_norm ? u * d : 2 * n_qk * d + (u - 2 * n_qk) * dv;
    const T* x = proj + qkv_off;
    float ss = 0.f;
    for (int j = lane; j < width; j += 32) {
        const int c = c0 + j;
        float acc = 0.f;
        for (int k = 0; k < taps; ++k)
            acc = fmaf(conv_w[(size_t)c * taps + k], conv_input<T>(x, stride, row0, li - (taps - 1 - k), c, C, tail, taps, fresh), acc);
        const float y = silu_f(acc);
        ss = fmaf(y, y, ss);
        arow[c] = y;
    }
    if (unit_norm) {                               // every lane scales what it wrote itself
        ss = warp_sum(ss);
        const float r = (u < n_qk ? q_scale : 1.0f) / sqrtf(ss + unit_eps);
        for (int j = lane; j < width; j += 32) arow[c0 + j] *= r;
    }
}

constexpr int COLS = 16, SLICES = 16, MAX_E = 32;
constexpr int THREADS = COLS * SLICES;

// E = entries of a column that one thread holds (a multiple of 4; thread `slice` owns slice * E .. + E - 1).
template <typename T, int E>
__global__ __launch_bounds__(THREADS) void delta_scan_kernel(
    const float* __restrict__ act, float* __restrict__ out, float* __restrict__ state, long long state_stride,
    long long tail_off, const T* __restrict__ proj, long long stride, int qkv_off, Seqs sq,
    int nh, int n_qk, int d, int dv, int taps) {
    pdl_wait();     // (the next kernel is let in at the end: this one runs long on few warps)
    constexpr int TOK = E > 8 ? 8 : 16;
    constexpr int DP = SLICES * E;
    constexpr int ES = E + 4;                      // shares sit 4 floats apart: no bank conflicts
    constexpr int DPS = SLICES * ES;
    __shared__ __align__(16) float qs[TOK * DPS];
    __shared__ __align__(16) float ks[TOK * DPS];
    __shared__ float vs[TOK * COLS];
    __shared__ float bg[TOK * 2];
    __shared__ __align__(16) float os[TOK * COLS * SLICES];
    const int b = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * COLS;
    const int row0 = sq.cu_seqlens[b], n = sq.cu_seqlens[b + 1] - row0;
    const int slice = threadIdx.x % SLICES, col = threadIdx.x / SLICES;
    const bool live = c0 + col < dv;
    const bool fresh = sq.ctx_lens[b] - n == 0;
    float* slot = state + (size_t)sq.state_slots[b] * state_stride;
    const int C = 2 * n_qk * d + nh * dv;
    const int AW = C + 2 * nh;
    if (taps > 1) {
        // the tail of the convolution after this step: the last taps - 1 inputs of the request, the channels
        // shared out among the request's CTAs (a channel's old tail is read by the thread that replaces it)
        float* tail = slot + tail_off;
        const T* x = proj + qkv_off;
        for (int c = (h * gridDim.z + blockIdx.z) * THREADS + threadIdx.x; c < C; c += nh * gridDim.z * THREADS) {
            float nv[MAX_TAPS - 1];
#pragma unroll
            for (int j = 0; j < MAX_TAPS - 1; ++j)
                nv[j] = j < taps - 1 ? conv_input<T>(x, stride, row0, n - (taps - 1) + j, c, C, tail, taps, fresh) : 0.f;
#pragma unroll
            for (int j = 0; j < MAX_TAPS - 1; ++j)
                if (j < taps - 1) tail[(size_t)j * C + c] = nv[j];
        }
    }
    float* S = slot + ((size_t)h * dv + c0 + col) * d;     // this thread's column: d contiguous entries
    const int hq = h / (nh / n_qk);
    float s[E];
#pragma unroll
    for (int e = 0; e < E; ++e) {
        const int i = slice * E + e;
        s[e] = (!fresh && live && i < d) ? S[i] : 0.f;
    }
    constexpr int PER = TOK * DP / THREADS;
    float rq[PER], rk[PER], rv;
    float rb = 0.f;
    auto fetch = [&](int t0) {
        const int nt = min(TOK, n - t0);
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int idx = threadIdx.x + j * THREADS, tt = idx / DP, i = idx - tt * DP;
            const bool ok = tt < nt && i < d;
            const float* r = act + (size_t)(row0 + t0 + (ok ? tt : 0)) * AW + hq * d + (ok ? i : 0);
            rq[j] = ok ? r[0] : 0.f;
            rk[j] = ok ? r[n_qk * d] : 0.f;
        }
        {
            const int tt = threadIdx.x / COLS, c = threadIdx.x - tt * COLS;     // TOK * COLS <= THREADS
            const bool ok = tt < nt && c0 + c < dv;
            rv = ok ? act[(size_t)(row0 + t0 + tt) * AW + 2 * n_qk * d + h * dv + c0 + c] : 0.f;
        }
        if (threadIdx.x < 2 * TOK) {
            const int tt = threadIdx.x >> 1, which = threadIdx.x & 1;
            rb = tt < nt ? act[(size_t)(row0 + t0 + tt) * AW + C + which * nh + h] : 0.f;
            if (which) rb = expf(rb);       // g from ln g
        }
    };
    if (n > 0) fetch(0);
    for (int t0 = 0; t0 < n; t0 += TOK) {
        const int nt = min(TOK, n - t0);
        __syncthreads();
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int idx = threadIdx.x + j * THREADS, tt = idx / DP, i = idx - tt * DP;
            const int at = tt * DPS + (i / E) * ES + i % E;
            qs[at] = rq[j];
            ks[at] = rk[j];
        }
        if (threadIdx.x < TOK * COLS) vs[threadIdx.x] = rv;
        if (threadIdx.x < 2 * TOK) bg[threadIdx.x] = rb;
        __syncthreads();
        if (t0 + TOK < n) fetch(t0 + TOK);
#pragma unroll 2
        for (int tt = 0; tt < nt; ++tt) {
            const float v = vs[tt * COLS + col];
            const float beta = bg[2 * tt], g = bg[2 * tt + 1];
            const float4* kr = reinterpret_cast<const float4*>(ks + tt * DPS + slice * ES);
            const float4* qr = reinterpret_cast<const float4*>(qs + tt * DPS + slice * ES);
            float4 k4[E / 4];
            float p[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int e4 = 0; e4 < E / 4; ++e4) {
                k4[e4] = kr[e4];
                p[0] = fmaf(s[4 * e4 + 0], k4[e4].x, p[0]);
                p[1] = fmaf(s[4 * e4 + 1], k4[e4].y, p[1]);
                p[2] = fmaf(s[4 * e4 + 2], k4[e4].z, p[2]);
                p[3] = fmaf(s[4 * e4 + 3], k4[e4].w, p[3]);
            }
            float dot = (p[0] + p[1]) + (p[2] + p[3]);
#pragma unroll
            for (int o = SLICES / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);    // the column's 16 threads
            const float u = beta * (v - g * dot);       // S^T k of the decayed state is g times that of the old one
            float o4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int e4 = 0; e4 < E / 4; ++e4) {
                const float4 q4 = qr[e4];
                s[4 * e4 + 0] = fmaf(g, s[4 * e4 + 0], k4[e4].x * u);
                s[4 * e4 + 1] = fmaf(g, s[4 * e4 + 1], k4[e4].y * u);
                s[4 * e4 + 2] = fmaf(g, s[4 * e4 + 2], k4[e4].z * u);
                s[4 * e4 + 3] = fmaf(g, s[4 * e4 + 3], k4[e4].w * u);
                o4[0] = fmaf(s[4 * e4 + 0], q4.x, o4[0]);
                o4[1] = fmaf(s[4 * e4 + 1], q4.y, o4[1]);
                o4[2] = fmaf(s[4 * e4 + 2], q4.z, o4[2]);
                o4[3] = fmaf(s[4 * e4 + 3], q4.w, o4[3]);
            }
            os[(tt * COLS + col) * SLICES + slice] = (o4[0] + o4[1]) + (o4[2] + o4[3]);
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < nt * COLS; idx += THREADS) {
            const int tt = idx / COLS, c = idx - tt * COLS;
            const float4* p4 = reinterpret_cast<const float4*>(os + idx * SLICES);
            float sum = 0.f;
#pragma unroll
            for (int j = 0; j < SLICES / 4; ++j) {
                const float4 a = p4[j];
                sum += (a.x + a.y) + (a.z + a.w);
            }
            if (c0 + c < dv) out[(size_t)(row0 + t0 + tt) * nh * dv + h * dv + c0 + c] = sum;
        }
    }
    if (live) {
#pragma unroll
        for (int e = 0; e < E; ++e) {
            const int i = slice * E + e;
            if (i < d) S[i] = s[e];
        }
    }
    pdl_trigger();
}

// ---- steps with prompts: 16 tokens at a time ------------------------------------------------------------------
constexpr int CH = 16;                 // tokens a chunk; equal to SLICES, so thread t of a column takes token t
constexpr int MS = CH + 4;             // row stride of the chunk's 16 x 16 matrices: rows read by 16-byte loads
constexpr int GRAM_WARPS = 4;

// gram[t][hq][0][j] = k_t . k_{t-j},  gram[t][hq][1][j] = q_t . k_{t-j}  for the tokens t - j of t's own chunk
// (chunks count from the first row of the request's portion); entries of other chunks are left as they are.
__global__ __launch_bounds__(GRAM_WARPS * 32) void delta_gram_kernel(
    const float* __restrict__ act, float* __restrict__ gram, Seqs sq, int n_units, int nh, int n_qk, int d, int dv) {
    pdl_wait();     // no early trigger: the chunk kernel's few CTAs are to find the SMs empty, one each
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int unit = blockIdx.x * GRAM_WARPS + warp;
    if (unit >= n_units) return;
    const int t = unit / n_qk, hq = unit - t * n_qk;
    const int b = sq.seq_of_token[t];
    const int back = (t - sq.cu_seqlens[b]) & (CH - 1);
    const int AW = 2 * n_qk * d + nh * dv + 2 * nh;
    const float* qt = act + (size_t)t * AW + hq * d;
    const float* kt = qt + n_qk * d;
    float qr[MAX_D / 32], kr[MAX_D / 32];
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) {
        const int e = lane + 32 * i;
        qr[i] = e < d ? qt[e] : 0.f;
        kr[i] = e < d ? kt[e] : 0.f;
    }
    float* g = gram + (size_t)t * (n_qk * 2 * CH + nh * CH) + hq * 2 * CH;
    for (int j = 0; j <= back; ++j) {
        const float* ki = kt - (size_t)j * AW;
        float a = 0.f, c = 0.f;
#pragma unroll
        for (int i = 0; i < MAX_D / 32; ++i) {
            const int e = lane + 32 * i;
            const float kv = e < d ? ki[e] : 0.f;
            a = fmaf(kr[i], kv, a);
            c = fmaf(qr[i], kv, c);
        }
        a = warp_sum(a);
        c = warp_sum(c);
        if (lane == 0) {
            g[j] = a;
            g[CH + j] = c;
        }
    }
}

// w[t][h][i] = row (t's place in its chunk) of (I + M)^-1 for the chunk's matrix M[a][i] = beta_a e^{L_a - L_i}
// k_a . k_i (i < a), so that the chunk's u are W (beta (v - e^L S0^T k)): a triangular system solved once a
// (token, head) for all columns, and for all chunks at once, outside the kernel that walks the chunks in order.
// One warp a (token, head): lane j keeps column j of the rows so far; row a = e_a - sum_{i<a} M[a][i] row_i.
__global__ __launch_bounds__(GRAM_WARPS * 32) void delta_solve_kernel(
    const float* __restrict__ act, float* __restrict__ gram, Seqs sq, int n_units, int nh, int n_qk, int d, int dv) {
    pdl_wait();     // no early trigger: the chunk kernel's few CTAs are to find the SMs empty, one each
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int unit = blockIdx.x * GRAM_WARPS + warp;
    if (unit >= n_units) return;
    const int t = unit / nh, h = unit - t * nh;
    const int hq = h / (nh / n_qk);
    const int b = sq.seq_of_token[t];
    const int back = (t - sq.cu_seqlens[b]) & (CH - 1);
    const int C = 2 * n_qk * d + nh * dv;
    const int AW = C + 2 * nh, GW = n_qk * 2 * CH + nh * CH;
    const int r0 = t - back;                        // the chunk's first row
    const int j = lane & (CH - 1);
    const bool in = j <= back;
    const float* arow = act + (size_t)(r0 + (in ? j : 0)) * AW + C;
    const float beta = in ? arow[h] : 0.f;
    float L = in ? arow[nh + h] : 0.f;
#pragma unroll
    for (int o = 1; o < CH; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, L, o, CH);
        if (j >= o) L += up;
    }
    float col[CH], kk[CH];                          // col[a] = W[a][j];  kk[a] = k_a . k_j
#pragma unroll
    for (int a = 0; a < CH; ++a)
        kk[a] = j < a && a <= back ? gram[(size_t)(r0 + a) * GW + hq * 2 * CH + (a - j)] : 0.f;
#pragma unroll
    for (int a = 0; a < CH; ++a) {
        col[a] = 0.f;
        if (a <= back) {                            // the same for the whole warp
            // lane i < a: M[a][i]
            const float La = __shfl_sync(0xffffffffu, L, a), ba = __shfl_sync(0xffffffffu, beta, a);
            const float mi = j < a ? ba * expf(La - L) * kk[a] : 0.f;
            float acc = j == a ? 1.f : 0.f;
#pragma unroll
            for (int i = 0; i < a; ++i) acc = fmaf(-__shfl_sync(0xffffffffu, mi, i), col[i], acc);
            col[a] = acc;
        }
    }
    float mine = 0.f;
#pragma unroll
    for (int a = 0; a < CH; ++a) mine = a == back ? col[a] : mine;
    if (lane < CH) gram[(size_t)t * GW + n_qk * 2 * CH + h * CH + j] = in ? mine : 0.f;
}

// Sums a[0..15] over the 16 lanes of a half-warp; lane `slice` returns the sum of index `slice`.  Halving
// exchanges: 8 + 4 + 2 + 1 shuffles, always the same order of additions.
__device__ __forceinline__ float reduce_scatter16(float (&a)[CH], int slice) {
#pragma unroll
    for (int off = CH / 2; off >= 1; off >>= 1) {
        const bool up = (slice & off) != 0;
#pragma unroll
        for (int m = 0; m < off; ++m) {
            const float send = up ? a[m] : a[m + off];
            const float keep = up ? a[m + off] : a[m];
            a[m] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
    }
    return a[0];
}

constexpr size_t chunk_smem_floats(int E) {
    return (size_t)2 * CH * SLICES * (E + 4) + CH * COLS + 2 * CH * MS + 4 * CH + COLS * (CH + 1);
}

constexpr int NC = 2;                          // columns a thread: a share of k or q read once serves both
constexpr int CGROUPS = COLS / NC;             // thread (slice, cg) holds columns cg and cg + CGROUPS
constexpr int CTHREADS = SLICES * CGROUPS;
constexpr int FT = CTHREADS / SLICES;          // tokens that the CTA's threads stage at a time

template <typename T, int E>
__global__ __launch_bounds__(CTHREADS) void delta_chunk_kernel(
    const float* __restrict__ act, const float* __restrict__ gram, float* __restrict__ out, float* __restrict__ state,
    long long state_stride, long long tail_off, const T* __restrict__ proj, long long stride, int qkv_off, Seqs sq,
    int nh, int n_qk, int d, int dv, int taps) {
    pdl_wait();     // (the next kernel is let in at the end: this one runs long on few warps)
    constexpr int ES = E + 4;                      // shares sit 4 floats apart: no bank conflicts
    constexpr int DPS = SLICES * ES;
    constexpr bool AHEAD = E <= 8;                 // the next chunk's rows wait in registers while this one runs
    constexpr int GRP = E <= 8 ? 4 : 1;            // tokens whose shares are loaded before the arithmetic on them
    constexpr int NF = CH / FT;
    extern __shared__ __align__(16) float sm[];
    float* qs = sm;                                // [CH][DPS]
    float* ks = qs + CH * DPS;                     // [CH][DPS]
    float* vs = ks + CH * DPS;                     // [CH][COLS]
    float* Ws = vs + CH * COLS;                    // [CH][MS] (I + M)^-1, see delta_solve_kernel
    float* Bs = Ws + CH * MS;                      // [CH][MS] e^{L_t - L_i} q_t . k_i, i <= t, else 0
    float* eL = Bs + CH * MS;                      // [CH] e^{L_t}
    float* wL = eL + CH;                           // [CH] e^{L_15 - L_t}
    float* bs = wL + CH;                           // [CH] beta_t
    float* Ls = bs + CH;                           // [CH] L_t
    float* os = Ls + CH;                           // [COLS][CH + 1]
    const int b = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * COLS;
    const int row0 = sq.cu_seqlens[b], n = sq.cu_seqlens[b + 1] - row0;
    const int slice = threadIdx.x % SLICES, cg = threadIdx.x / SLICES;
    const bool fresh = sq.ctx_lens[b] - n == 0;
    float* slot = state + (size_t)sq.state_slots[b] * state_stride;
    const int C = 2 * n_qk * d + nh * dv;
    const int AW = C + 2 * nh, GW = n_qk * 2 * CH + nh * CH;
    if (taps > 1) {
        // the tail of the convolution after this step: the last taps - 1 inputs of the request, the channels
        // shared out among the request's CTAs (a channel's old tail is read by the thread that replaces it)
        float* tail = slot + tail_off;
        const T* x = proj + qkv_off;
        for (int c = (h * gridDim.z + blockIdx.z) * CTHREADS + threadIdx.x; c < C; c += nh * gridDim.z * CTHREADS) {
            float nv[MAX_TAPS - 1];
#pragma unroll
            for (int j = 0; j < MAX_TAPS - 1; ++j)
                nv[j] = j < taps - 1 ? conv_input<T>(x, stride, row0, n - (taps - 1) + j, c, C, tail, taps, fresh) : 0.f;
#pragma unroll
            for (int j = 0; j < MAX_TAPS - 1; ++j)
                if (j < taps - 1) tail[(size_t)j * C + c] = nv[j];
        }
    }
    const int hq = h / (nh / n_qk);
    float* S[NC];                                  // this thread's columns: d contiguous entries each
    bool live[NC];
    float s[NC][E];
#pragma unroll
    for (int x = 0; x < NC; ++x) {
        live[x] = c0 + cg + x * CGROUPS < dv;
        S[x] = slot + ((size_t)h * dv + c0 + cg + x * CGROUPS) * d;
#pragma unroll
        for (int e = 0; e < E; ++e) {
            const int i = slice * E + e;
            s[x][e] = (!fresh && live[x] && i < d) ? S[x][i] : 0.f;
        }
    }
    // What a thread brings to shared memory for a chunk, as thread (ft = tid / 16, fj = tid % 16), of the tokens ft,
    // ft + FT, ..: share fj of the token's q and k, its v of column fj, entry fj of its rows of W and of q . k; and in
    // warp 0 beta (lanes 0..15) or ln g (16..31) of token tid % 16.  A token past the portion's end: zeros, beta 0, g 1.
    const int ft = threadIdx.x / SLICES, fj = threadIdx.x % SLICES;
    float rq[NF][E], rk[NF][E], rv[NF], rw[NF], rgq[NF], rb = 0.f;
    auto fetch = [&](int t0) {
#pragma unroll
        for (int x = 0; x < NF; ++x) {
            const int tt = ft + x * FT;
            const bool tok = t0 + tt < n;
            const float* arow = act + (size_t)(row0 + t0 + (tok ? tt : 0)) * AW;
            const float* grow = gram + (size_t)(row0 + t0 + (tok ? tt : 0)) * GW;
#pragma unroll
            for (int e = 0; e < E; ++e) {
                const int i = fj * E + e;
                const bool ok = tok && i < d;
                rq[x][e] = ok ? arow[hq * d + i] : 0.f;
                rk[x][e] = ok ? arow[(n_qk + hq) * d + i] : 0.f;
            }
            rv[x] = tok && c0 + fj < dv ? arow[2 * n_qk * d + h * dv + c0 + fj] : 0.f;
            rw[x] = tok ? grow[n_qk * 2 * CH + h * CH + fj] : 0.f;
            rgq[x] = tok && fj <= tt ? grow[hq * 2 * CH + CH + fj] : 0.f;
        }
        if (threadIdx.x < 2 * CH) {
            const int tt = threadIdx.x & (CH - 1), which = threadIdx.x >> 4;
            rb = t0 + tt < n ? act[(size_t)(row0 + t0 + tt) * AW + C + which * nh + h] : 0.f;
        }
    };
    if (AHEAD && n > 0) fetch(0);
    for (int t0 = 0; t0 < n; t0 += CH) {
        const int nt = min(CH, n - t0);
        __syncthreads();
        if (!AHEAD) fetch(t0);
#pragma unroll
        for (int x = 0; x < NF; ++x) {
            const int tt = ft + x * FT;
            float4* q4 = reinterpret_cast<float4*>(qs + tt * DPS + fj * ES);
            float4* k4 = reinterpret_cast<float4*>(ks + tt * DPS + fj * ES);
#pragma unroll
            for (int e4 = 0; e4 < E / 4; ++e4) {
                q4[e4] = make_float4(rq[x][4 * e4], rq[x][4 * e4 + 1], rq[x][4 * e4 + 2], rq[x][4 * e4 + 3]);
                k4[e4] = make_float4(rk[x][4 * e4], rk[x][4 * e4 + 1], rk[x][4 * e4 + 2], rk[x][4 * e4 + 3]);
            }
            vs[tt * COLS + fj] = rv[x];
            Ws[tt * MS + fj] = rw[x];
        }
        if (threadIdx.x < 32) {
            float L = rb;                           // lanes 16..31: running sum of ln g
#pragma unroll
            for (int o = 1; o < CH; o <<= 1) {
                const float up = __shfl_up_sync(0xffffffffu, L, o, CH);
                if ((threadIdx.x & (CH - 1)) >= o) L += up;
            }
            const float last = __shfl_sync(0xffffffffu, L, 31);
            if (threadIdx.x < CH) bs[threadIdx.x] = rb;
            else {
                const int tt = threadIdx.x - CH;
                Ls[tt] = L;
                eL[tt] = expf(L);
                wL[tt] = expf(last - L);
            }
        }
        __syncthreads();
#pragma unroll
        for (int x = 0; x < NF; ++x) {
            const int tt = ft + x * FT, i = tt - fj;                  // fj tokens back
            if (i >= 0) Bs[tt * MS + i] = expf(Ls[tt] - Ls[i]) * rgq[x];
            else Bs[tt * MS + CH + i] = 0.f;
        }
        if (AHEAD && t0 + CH < n) fetch(t0 + CH);
        // S0^T k_t and S0^T q_t of the 16 tokens: this thread's share, then the sum over the column's threads
        float pk[NC][CH], pq[NC][CH];
#pragma unroll
        for (int tt0 = 0; tt0 < CH; tt0 += GRP) {
            float4 kk[GRP][E / 4], qq[GRP][E / 4];
#pragma unroll
            for (int g = 0; g < GRP; ++g) {
                const float4* kr = reinterpret_cast<const float4*>(ks + (tt0 + g) * DPS + slice * ES);
                const float4* qr = reinterpret_cast<const float4*>(qs + (tt0 + g) * DPS + slice * ES);
#pragma unroll
                for (int e4 = 0; e4 < E / 4; ++e4) kk[g][e4] = kr[e4], qq[g][e4] = qr[e4];
            }
#pragma unroll
            for (int g = 0; g < GRP; ++g) {
#pragma unroll
                for (int x = 0; x < NC; ++x) {
                    float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll
                    for (int e4 = 0; e4 < E / 4; ++e4) {
                        a0 = fmaf(s[x][4 * e4 + 0], kk[g][e4].x, a0);
                        a1 = fmaf(s[x][4 * e4 + 1], kk[g][e4].y, a1);
                        a0 = fmaf(s[x][4 * e4 + 2], kk[g][e4].z, a0);
                        a1 = fmaf(s[x][4 * e4 + 3], kk[g][e4].w, a1);
                        b0 = fmaf(s[x][4 * e4 + 0], qq[g][e4].x, b0);
                        b1 = fmaf(s[x][4 * e4 + 1], qq[g][e4].y, b1);
                        b0 = fmaf(s[x][4 * e4 + 2], qq[g][e4].z, b0);
                        b1 = fmaf(s[x][4 * e4 + 3], qq[g][e4].w, b1);
                    }
                    pk[x][tt0 + g] = a0 + a1;
                    pq[x][tt0 + g] = b0 + b1;
                }
            }
        }
        float sk[NC], sqt[NC];
#pragma unroll
        for (int x = 0; x < NC; ++x) {
            sk[x] = reduce_scatter16(pk[x], slice);        // token `slice`'s
            sqt[x] = reduce_scatter16(pq[x], slice);
        }
        __syncthreads();                                   // Bs is written
        const int t = slice;
        const float el = eL[t], bt = bs[t];
        float u[NC][CH];
        {
            // u_t = sum_i W[t][i] r_i, then every thread of the column takes all 16
            float w[CH];
            const float4* wr = reinterpret_cast<const float4*>(Ws + t * MS);
#pragma unroll
            for (int j = 0; j < CH / 4; ++j) {
                const float4 a = wr[j];
                w[4 * j] = a.x, w[4 * j + 1] = a.y, w[4 * j + 2] = a.z, w[4 * j + 3] = a.w;
            }
#pragma unroll
            for (int x = 0; x < NC; ++x) {
                const float r = bt * (vs[t * COLS + cg + x * CGROUPS] - el * sk[x]);
                float u0 = 0.f, u1 = 0.f;
#pragma unroll
                for (int i = 0; i < CH; i += 2) {
                    u0 = fmaf(w[i], __shfl_sync(0xffffffffu, r, i, CH), u0);
                    u1 = fmaf(w[i + 1], __shfl_sync(0xffffffffu, r, i + 1, CH), u1);
                }
                const float ut = u0 + u1;
#pragma unroll
                for (int i = 0; i < CH; ++i) u[x][i] = __shfl_sync(0xffffffffu, ut, i, CH);
            }
        }
        {
            float bq[CH];
            const float4* br = reinterpret_cast<const float4*>(Bs + t * MS);
#pragma unroll
            for (int j = 0; j < CH / 4; ++j) {
                const float4 a = br[j];
                bq[4 * j] = a.x, bq[4 * j + 1] = a.y, bq[4 * j + 2] = a.z, bq[4 * j + 3] = a.w;
            }
#pragma unroll
            for (int x = 0; x < NC; ++x) {
                float o0 = el * sqt[x], o1 = 0.f;
#pragma unroll
                for (int i = 0; i < CH; i += 2) {
                    o0 = fmaf(bq[i], u[x][i], o0);
                    o1 = fmaf(bq[i + 1], u[x][i + 1], o1);
                }
                os[(cg + x * CGROUPS) * (CH + 1) + t] = o0 + o1;
            }
        }
        {
            const float dec = eL[CH - 1];
            const float4* wr = reinterpret_cast<const float4*>(wL);
#pragma unroll
            for (int j = 0; j < CH / 4; ++j) {
                const float4 a = wr[j];
#pragma unroll
                for (int x = 0; x < NC; ++x)
                    u[x][4 * j] *= a.x, u[x][4 * j + 1] *= a.y, u[x][4 * j + 2] *= a.z, u[x][4 * j + 3] *= a.w;
            }
#pragma unroll
            for (int x = 0; x < NC; ++x)
#pragma unroll
                for (int e = 0; e < E; ++e) s[x][e] *= dec;
#pragma unroll
            for (int tt0 = 0; tt0 < CH; tt0 += GRP) {
                float4 kk[GRP][E / 4];
#pragma unroll
                for (int g = 0; g < GRP; ++g) {
                    const float4* kr = reinterpret_cast<const float4*>(ks + (tt0 + g) * DPS + slice * ES);
#pragma unroll
                    for (int e4 = 0; e4 < E / 4; ++e4) kk[g][e4] = kr[e4];
                }
#pragma unroll
                for (int g = 0; g < GRP; ++g) {
#pragma unroll
                    for (int x = 0; x < NC; ++x) {
#pragma unroll
                        for (int e4 = 0; e4 < E / 4; ++e4) {
                            s[x][4 * e4 + 0] = fmaf(kk[g][e4].x, u[x][tt0 + g], s[x][4 * e4 + 0]);
                            s[x][4 * e4 + 1] = fmaf(kk[g][e4].y, u[x][tt0 + g], s[x][4 * e4 + 1]);
                            s[x][4 * e4 + 2] = fmaf(kk[g][e4].z, u[x][tt0 + g], s[x][4 * e4 + 2]);
                            s[x][4 * e4 + 3] = fmaf(kk[g][e4].w, u[x][tt0 + g], s[x][4 * e4 + 3]);
                        }
                    }
                }
            }
        }
        __syncthreads();
#pragma unroll
        for (int x = 0; x < NF; ++x) {
            const int tt = ft + x * FT;
            if (tt < nt && c0 + fj < dv) out[(size_t)(row0 + t0 + tt) * nh * dv + h * dv + c0 + fj] = os[fj * (CH + 1) + tt];
        }
    }
#pragma unroll
    for (int x = 0; x < NC; ++x) {
        if (!live[x]) continue;
#pragma unroll
        for (int e = 0; e < E; ++e) {
            const int i = slice * E + e;
            if (i < d) S[x][i] = s[x][e];
        }
    }
    pdl_trigger();
}
}  // namespace

// Floats of a request's state slot: S of every head, then the convolution's tail.
extern "C" int rlis_gated_delta_state_floats(int nh, int n_qk, int d, int dv, int taps) {
    return nh * dv * d + (taps - 1) * (2 * n_qk * d + nh * dv);
}

// proj [T, stride] in the element type: q | k | v columns from qkv_off (n_qk heads of d, n_qk of d, nh of dv),
// nh logits of beta from b_off and of the decay from a_off.  conv_w float32 [C, taps] in the same channel order.
// state float32 [slots, state_stride]; act float32 [T, C + 2 nh] (scratch); out float32 [T, nh dv].
// gram: null for the token-by-token kernel (steps of single tokens and short portions), else float32
// [T, n_qk * 32 + nh * 16] of scratch for the kernels that take 16 tokens at a time.
extern "C" int rlis_gated_delta(const void* proj, long long stride, int qkv_off, int b_off, int a_off,
                                const float* conv_w, const float* a_log, const float* dt_bias, float* state,
                                long long state_stride, const int* cu_seqlens, const int* ctx_lens,
                                const int* state_slots, const int* seq_of_token, float* act, float* gram, float* out,
                                int n_tokens, int n_seqs, int nh, int n_qk, int d, int dv, int taps, float unit_eps,
                                float q_scale, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return 0;
    if (d <= 0 || d > MAX_D || d > SLICES * MAX_E || dv <= 0 || dv > MAX_D || nh <= 0 || nh > 65535 || n_qk <= 0 ||
        nh % n_qk != 0 || taps < 1 || taps > MAX_TAPS)
        return RLIS_ERR_UNSUPPORTED;
    const long long tail_off = (long long)nh * dv * d;
    if (state_stride < rlis_gated_delta_state_floats(nh, n_qk, d, dv, taps)) return RLIS_ERR_UNSUPPORTED;
    const long long units = (long long)n_tokens * (2 * n_qk + nh + 1);
    if (units > 0x7fffffffLL) return RLIS_ERR_UNSUPPORTED;
    const Seqs sq{cu_seqlens, ctx_lens, state_slots, seq_of_token};
    const unsigned pblocks = (unsigned)((units + PREP_WARPS - 1) / PREP_WARPS);
    dim3 grid(n_seqs, nh, (dv + COLS - 1) / COLS);
    const int e = (d + SLICES - 1) / SLICES;
    const int gunits = n_tokens * n_qk, sunits = n_tokens * nh;
    // few CTAs that run long: shared memory asked for beyond the need keeps them one an SM
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    }
    const bool spread = (long long)grid.x * grid.y * grid.z <= sms;
#define RLIS_DELTA(T, E)                                                                                                 \
    do {                                                                                                                 \
        const size_t bytes = spread && n_tokens > n_seqs ? 120 * 1024 : 0;                                               \
        if (bytes) cudaFuncSetAttribute(delta_scan_kernel<T, E>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes); \
        rlis_launch(delta_scan_kernel<T, E>, grid, THREADS, bytes, stream, act, out, state, state_stride, tail_off,      \
                    (const T*)proj, stride, qkv_off, sq, nh, n_qk, d, dv, taps);                                         \
    } while (0)
#define RLIS_CHUNK(T, E)                                                                                                 \
    do {                                                                                                                 \
        size_t bytes = chunk_smem_floats(E) * sizeof(float);                                                             \
        if (spread && bytes < 120 * 1024) bytes = 120 * 1024;                                                            \
        cudaFuncSetAttribute(delta_chunk_kernel<T, E>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);         \
        rlis_launch(delta_chunk_kernel<T, E>, grid, CTHREADS, bytes, stream, act, (const float*)gram, out, state,         \
                    state_stride, tail_off, (const T*)proj, stride, qkv_off, sq, nh, n_qk, d, dv, taps);                 \
    } while (0)
#define RLIS_DELTA_T(T)                                                                                                  \
    do {                                                                                                                 \
        rlis_launch(delta_prepare_kernel<T>, pblocks, PREP_WARPS * 32, 0, stream, (const T*)proj, stride, qkv_off,       \
                    b_off, a_off, conv_w, a_log, dt_bias, (const float*)state, state_stride, tail_off, sq, act,          \
                    (int)units, nh, n_qk, d, dv, taps, unit_eps, q_scale);                                               \
        if (gram) {                                                                                                      \
            rlis_launch(delta_gram_kernel, (unsigned)((gunits + GRAM_WARPS - 1) / GRAM_WARPS), GRAM_WARPS * 32, 0,       \
                        stream, (const float*)act, gram, sq, gunits, nh, n_qk, d, dv);                                   \
            rlis_launch(delta_solve_kernel, (unsigned)((sunits + GRAM_WARPS - 1) / GRAM_WARPS), GRAM_WARPS * 32, 0,      \
                        stream, (const float*)act, gram, sq, sunits, nh, n_qk, d, dv);                                   \
            if (e <= 4) RLIS_CHUNK(T, 4);                                                                                \
            else if (e <= 8) RLIS_CHUNK(T, 8);                                                                           \
            else if (e <= 16) RLIS_CHUNK(T, 16);                                                                         \
            else RLIS_CHUNK(T, 32);                                                                                      \
        } else if (e <= 4) RLIS_DELTA(T, 4);                                                                             \
        else if (e <= 8) RLIS_DELTA(T, 8);                                                                               \
        else if (e <= 16) RLIS_DELTA(T, 16);                                                                             \
        else RLIS_DELTA(T, 32);                                                                                          \
    } while (0)
    if (dtype == RLIS_F32) RLIS_DELTA_T(float);
    else if (dtype == RLIS_BF16) RLIS_DELTA_T(bf16);
    else return RLIS_ERR_UNSUPPORTED;
#undef RLIS_DELTA_T
#undef RLIS_CHUNK
#undef RLIS_DELTA
    return RLIS_LAUNCH_CHECK();
}

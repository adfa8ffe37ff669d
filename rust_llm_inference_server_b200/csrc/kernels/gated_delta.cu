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
// prepare: one warp a (token, head of q, k or v), and one more a token for beta and g; writes float32 rows
//          [q | k | v | beta | g].  It reads the convolution's tail from the slot and leaves it as it is.
// scan:    columns of S evolve independently: a CTA takes (request, head, 16 columns), 16 threads share a column
//          (each a contiguous share of its entries in registers) and walk the request's tokens of this step in
//          order; the column's dot product with k is summed over the 16 threads by shuffles, the read-out's
//          partial sums after each tile of tokens.  The CTA of head 0, columns 0 also moves the slot's
//          convolution tail on (after every reader of the old one is done: the prepare kernel has finished).
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
            arow[C + nh + h] = expf(-expf(a_log[h]) * softplus_f(to_f<T>(row[a_off + h]) + dt_bias[h]));
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
    float y[MAX_D / 32];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) {
        const int j = lane + 32 * i;
        y[i] = 0.f;
        if (j < width) {
            const int c = c0 + j;
            float acc = 0.f;
            for (int k = 0; k < taps; ++k)
                acc = fmaf(conv_w[(size_t)c * taps + k], conv_input<T>(x, stride, row0, li - (taps - 1 - k), c, C, tail, taps, fresh), acc);
            y[i] = silu_f(acc);
            ss = fmaf(y[i], y[i], ss);
        }
    }
    float r = 1.0f;
    if (unit_norm) {
        ss = warp_sum(ss);
        r = (u < n_qk ? q_scale : 1.0f) / sqrtf(ss + unit_eps);
    }
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) {
        const int j = lane + 32 * i;
        if (j < width) arow[c0 + j] = y[i] * r;
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
    if (h == 0 && blockIdx.z == 0 && taps > 1) {
        // the tail of the convolution after this step: the last taps - 1 inputs of the request
        float* tail = slot + tail_off;
        const T* x = proj + qkv_off;
        for (int c = threadIdx.x; c < C; c += THREADS) {
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
}  // namespace

// Floats of a request's state slot: S of every head, then the convolution's tail.
extern "C" int rlis_gated_delta_state_floats(int nh, int n_qk, int d, int dv, int taps) {
    return nh * dv * d + (taps - 1) * (2 * n_qk * d + nh * dv);
}

// proj [T, stride] in the element type: q | k | v columns from qkv_off (n_qk heads of d, n_qk of d, nh of dv),
// nh logits of beta from b_off and of the decay from a_off.  conv_w float32 [C, taps] in the same channel order.
// state float32 [slots, state_stride]; act float32 [T, C + 2 nh] (scratch); out float32 [T, nh dv].
extern "C" int rlis_gated_delta(const void* proj, long long stride, int qkv_off, int b_off, int a_off,
                                const float* conv_w, const float* a_log, const float* dt_bias, float* state,
                                long long state_stride, const int* cu_seqlens, const int* ctx_lens,
                                const int* state_slots, const int* seq_of_token, float* act, float* out, int n_tokens,
                                int n_seqs, int nh, int n_qk, int d, int dv, int taps, float unit_eps, float q_scale,
                                int dtype, cudaStream_t stream) {
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
#define RLIS_DELTA(T, E) rlis_launch(delta_scan_kernel<T, E>, grid, THREADS, 0, stream, act, out, state, state_stride, \
                                     tail_off, (const T*)proj, stride, qkv_off, sq, nh, n_qk, d, dv, taps)
#define RLIS_DELTA_T(T)                                                                                                  \
    do {                                                                                                                 \
        rlis_launch(delta_prepare_kernel<T>, pblocks, PREP_WARPS * 32, 0, stream, (const T*)proj, stride, qkv_off,       \
                    b_off, a_off, conv_w, a_log, dt_bias, (const float*)state, state_stride, tail_off, sq, act,          \
                    (int)units, nh, n_qk, d, dv, taps, unit_eps, q_scale);                                               \
        if (e <= 4) RLIS_DELTA(T, 4);                                                                                    \
        else if (e <= 8) RLIS_DELTA(T, 8);                                                                               \
        else if (e <= 16) RLIS_DELTA(T, 16);                                                                             \
        else RLIS_DELTA(T, 32);                                                                                          \
    } while (0)
    if (dtype == RLIS_F32) RLIS_DELTA_T(float);
    else if (dtype == RLIS_BF16) RLIS_DELTA_T(bf16);
    else return RLIS_ERR_UNSUPPORTED;
#undef RLIS_DELTA_T
#undef RLIS_DELTA
    return RLIS_LAUNCH_CHECK();
}

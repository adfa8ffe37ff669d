// Linear attention with a per-head decay, as a recurrence over a float32 state:
//
//   q, k = silu(.) [heads, d]; v = silu(.) [heads, dv]           (from one fused projection's rows)
//   S_t = decay_h * S_(t-1) + k_t v_t^T ;  o_t = S_t^T q_t        S [d, dv] per request and head (stored transposed)
//
// The state of a request lives in its state slot between steps; a request whose first token is in
// this step starts from zero.  Columns of S evolve independently, so a CTA takes (request, head,
// 16 columns): 16 threads share a column, each holding a contiguous sixteenth of its entries in
// registers, and walk the request's tokens of this step in order; a column's partial sums are added
// after each tile of tokens.  The state is stored column by column, [slot, head, dv, d], so that a
// thread's entries are contiguous in memory.  Tokens are staged through shared
// memory 16 (or 8) at a time (silu applied once on the way in), the next 16 already on their way from
// global memory while the current ones are worked on.
// Everything after the projection is float32; the order of every sum depends on d only.
//
// The same walk serves recurrences whose decay differs by token and channel, S_t = diag(a_t) S_(t-1) + k_t v_t^T
// (VEC: a is staged like k, from columns a_off of the rows), and inputs that another kernel has prepared in
// float32 (`rlis_recurrence_inputs`: rotation of q and k by position, a scale on k, silu of q, a forget gate a = l +
// (1 - l) sigmoid(z + b) with k = 1 - a), through `rlis_recurrence_scan`.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int COLS = 16, SLICES = 16, MAX_E = 32;   // d up to 512
constexpr int THREADS = COLS * SLICES;

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

// What the walk needs to make its inputs itself in short steps (PREP 1: rotation by halves and a scale on k; PREP 2: silu
// of q and the forget gate); the arithmetic is that of recurrence_inputs_kernel below.
struct PrepArgs {
    const float* inv_freq;
    int rot_dims;
    float k_scale;
    const float* lower;
    const float* gate_bias;
};

// E = entries of a column that one thread holds: ceil(d / 8), rounded up to a multiple of 4 so that a
// thread reads its share of k and q from shared memory in 16-byte vectors.  Thread `slice` owns the
// entries slice * E .. slice * E + E - 1 (those at or beyond d stay zero).
// KCOMP (with VEC): the key is the complement of the decay, k = 1 - a, taken from the staged decays: two arrays as without a
// decay a channel, so a stage holds as many tokens.
template <typename T, int E, bool SILU, bool VEC, int PREP = 0, bool KCOMP = false>
__global__ __launch_bounds__(THREADS) void lightning_scan_kernel(
    const T* __restrict__ proj, long long stride, int q_off, int k_off, int v_off, float* __restrict__ out,
    float* __restrict__ state, const float* __restrict__ decay, const int* __restrict__ cu_seqlens,
    const int* __restrict__ ctx_lens, const int* __restrict__ state_slots, int nh, int d, int dv, int a_off,
    const PrepArgs pa) {
    pdl_wait();     // (the next kernel is let in at the end: this one runs long on few warps)
    // tokens staged at a time (shared memory holds them; a third array with a decay a channel)
    constexpr int TOK = VEC && !KCOMP ? (E > 16 ? 4 : 8) : (E > 8 ? 8 : 16);
    constexpr int DP = SLICES * E;                 // padded d
    constexpr int ES = E + 4;                      // a thread's share sits 4 floats apart from the next one's: no bank conflicts
    constexpr int DPS = SLICES * ES;
    __shared__ __align__(16) float qs[TOK * DPS];
    __shared__ __align__(16) float ks[KCOMP ? 4 : TOK * DPS];
    __shared__ __align__(16) float as[VEC ? TOK * DPS : 4];
    __shared__ float vs[TOK * COLS];
    __shared__ __align__(16) float os[TOK * COLS * SLICES];   // a column's sixteen partial sums a token
    const int b = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * COLS;
    const int row0 = cu_seqlens[b], n = cu_seqlens[b + 1] - row0;
    const int slice = threadIdx.x % SLICES, col = threadIdx.x / SLICES;
    const bool live = c0 + col < dv;
    const bool fresh = ctx_lens[b] - n == 0;      // the request starts in this step
    const int slot = state_slots[b];
    float* S = state + (((size_t)slot * nh + h) * dv + c0 + col) * d;    // this thread's column: d contiguous entries
    const float g = VEC ? 0.f : decay[h];
    float s[E];
    const bool quads = d % 4 == 0;                 // a thread's entries are then whole 16-byte vectors
    if (quads) {
#pragma unroll
        for (int e = 0; e < E; e += 4) {
            const int i = slice * E + e;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (!fresh && live && i < d) v = *reinterpret_cast<const float4*>(S + i);
            s[e] = v.x; s[e + 1] = v.y; s[e + 2] = v.z; s[e + 3] = v.w;
        }
    } else {
#pragma unroll
        for (int e = 0; e < E; ++e) {
            const int i = slice * E + e;
            s[e] = (!fresh && live && i < d) ? S[i] : 0.f;
        }
    }
    // what one thread stages of q and k: element idx = threadIdx.x + j * THREADS of the [TOK][DP] tile
    constexpr int PER = TOK * DP / THREADS;
    float rq[PER], rk[PER], ra[VEC && PREP != 2 ? PER : 1], rv[(TOK * COLS + THREADS - 1) / THREADS];
    float rqp[PREP == 1 ? PER : 1], rkp[PREP == 1 ? PER : 1];      // the entries that q and k turn with
    const int half = pa.rot_dims >> 1;
    const int pos0 = ctx_lens[b] - n;                              // position of the request's first token of this step
    auto fetch = [&](int t0) {                     // raw values of the next tokens, into registers
        const int nt = min(TOK, n - t0);
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int idx = threadIdx.x + j * THREADS, tt = idx / DP, i = idx - tt * DP;
            const bool ok = tt < nt && i < d;
            const T* r = proj + (size_t)(row0 + t0 + (ok ? tt : 0)) * stride + h * d + (ok ? i : 0);
            rq[j] = ok ? to_f<T>(r[q_off]) : 0.f;
            if (!KCOMP || PREP == 2) rk[j] = ok ? to_f<T>(r[k_off]) : 0.f;
            if (VEC && PREP != 2) ra[j] = ok ? to_f<T>(r[a_off]) : 0.f;
            if (PREP == 1) {
                const bool turns = ok && i < pa.rot_dims;
                const int pi = i < half ? half : -half;
                rqp[j] = turns ? to_f<T>(r[q_off + pi]) : 0.f;
                rkp[j] = turns ? to_f<T>(r[k_off + pi]) : 0.f;
            }
        }
#pragma unroll
        for (int j = 0; j < (TOK * COLS + THREADS - 1) / THREADS; ++j) {
            const int idx = threadIdx.x + j * THREADS, tt = idx / COLS, c = idx - tt * COLS;
            const bool ok = idx < TOK * COLS && tt < nt && c0 + c < dv;
            rv[j] = ok ? to_f<T>(proj[(size_t)(row0 + t0 + tt) * stride + v_off + h * dv + c0 + c]) : 0.f;
        }
    };
    if (n > 0) fetch(0);
    for (int t0 = 0; t0 < n; t0 += TOK) {
        const int nt = min(TOK, n - t0);
        __syncthreads();                           // the last tile's readers are done
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int idx = threadIdx.x + j * THREADS, tt = idx / DP, i = idx - tt * DP;
            const int at = tt * DPS + (i / E) * ES + i % E;
            if (PREP == 1) {
                float qv = rq[j], kv = rk[j];
                if (tt < nt && i < pa.rot_dims) {          // (a stage's empty places are zeros and stay so)
                    float sn, cs;
                    sincosf((float)(pos0 + t0 + tt) * pa.inv_freq[i < half ? i : i - half], &sn, &cs);
                    qv = i < half ? rope_first(qv, rqp[j], cs, sn) : rope_second(rqp[j], qv, cs, sn);
                    kv = i < half ? rope_first(kv, rkp[j], cs, sn) : rope_second(rkp[j], kv, cs, sn);
                }
                qs[at] = qv;
                ks[at] = kv * pa.k_scale;
            } else if (PREP == 2) {
                const bool ok = tt < nt && i < d;
                float a = 0.f;
                if (ok) {
                    const float l = pa.lower[h * d + i];
                    const float z = rk[j] + (pa.gate_bias != nullptr ? pa.gate_bias[h * d + i] : 0.f);
                    a = l + (1.0f - l) * (1.0f / (1.0f + expf(-z)));
                }
                qs[at] = silu_f(rq[j]);
                if (!KCOMP) ks[at] = ok ? 1.0f - a : 0.f;
                as[at] = KCOMP && !ok ? 1.0f : a;          // (an empty place keeps what it holds: a = 1, k = 0)
            } else {
                qs[at] = SILU ? silu_f(rq[j]) : rq[j];  // silu(0) = 0 keeps the padding zero
                if (!KCOMP) ks[at] = SILU ? silu_f(rk[j]) : rk[j];
                if (VEC) as[at] = KCOMP && !(tt < nt && i < d) ? 1.0f : ra[j];
            }
        }
#pragma unroll
        for (int j = 0; j < (TOK * COLS + THREADS - 1) / THREADS; ++j) {
            const int idx = threadIdx.x + j * THREADS;
            if (idx < TOK * COLS) vs[idx] = SILU ? silu_f(rv[j]) : rv[j];
        }
        __syncthreads();
        if (t0 + TOK < n) fetch(t0 + TOK);         // in flight while this tile is worked on
#pragma unroll 4
        for (int tt = 0; tt < nt; ++tt) {
            const float v = vs[tt * COLS + col];
            const float4* kr = reinterpret_cast<const float4*>(ks + (KCOMP ? 0 : tt * DPS + slice * ES));
            const float4* qr = reinterpret_cast<const float4*>(qs + tt * DPS + slice * ES);
            const float4* ar = reinterpret_cast<const float4*>(as + (VEC ? tt * DPS + slice * ES : 0));
            float o[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int e4 = 0; e4 < E / 4; ++e4) {
                const float4 q4 = qr[e4];
                const float4 a4 = VEC ? ar[e4] : make_float4(g, g, g, g);
                const float4 k4 = KCOMP ? make_float4(1.0f - a4.x, 1.0f - a4.y, 1.0f - a4.z, 1.0f - a4.w) : kr[e4];
                s[4 * e4 + 0] = fmaf(a4.x, s[4 * e4 + 0], k4.x * v);
                s[4 * e4 + 1] = fmaf(a4.y, s[4 * e4 + 1], k4.y * v);
                s[4 * e4 + 2] = fmaf(a4.z, s[4 * e4 + 2], k4.z * v);
                s[4 * e4 + 3] = fmaf(a4.w, s[4 * e4 + 3], k4.w * v);
                o[0] = fmaf(s[4 * e4 + 0], q4.x, o[0]);
                o[1] = fmaf(s[4 * e4 + 1], q4.y, o[1]);
                o[2] = fmaf(s[4 * e4 + 2], q4.z, o[2]);
                o[3] = fmaf(s[4 * e4 + 3], q4.w, o[3]);
            }
            // the partial sums of a column are added after the tile: no shuffle chain per token
            os[(tt * COLS + col) * SLICES + slice] = (o[0] + o[1]) + (o[2] + o[3]);
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
    if (live && quads) {
#pragma unroll
        for (int e = 0; e < E; e += 4) {
            const int i = slice * E + e;
            if (i < d) *reinterpret_cast<float4*>(S + i) = make_float4(s[e], s[e + 1], s[e + 2], s[e + 3]);
        }
    } else if (live) {
#pragma unroll
        for (int e = 0; e < E; ++e) {
            const int i = slice * E + e;
            if (i < d) S[i] = s[e];
        }
    }
    pdl_trigger();
}

// out[t, :] = silu(x[t, :width]) in float32: the activation applied once for every CTA of the scan
// that reads it (long steps; a short step applies it while staging).
template <typename T>
__global__ void silu_rows_kernel(const T* __restrict__ x, long long stride, float* __restrict__ out, int width) {
    // The scan that follows has few CTAs and wants one to an SM: let in early, while this grid still fills
    // the SMs, its CTAs would land several to an SM wherever room appears first.  So it is let in at the end.
    pdl_wait();
    const T* xr = x + (size_t)blockIdx.x * stride;
    float* orow = out + (size_t)blockIdx.x * width;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < width; c += gridDim.y * blockDim.x)
        orow[c] = silu_f(to_f<T>(xr[c]));
    pdl_trigger();
}

template <typename T, bool SILU, bool VEC = false, int PREP = 0, bool KCOMP = false>
int launch_scan(const T* proj, long long stride, int q_off, int k_off, int v_off, float* out, float* state,
                const float* decay, const int* cu, const int* ctx, const int* slots, dim3 grid, int nh, int d, int dv,
                cudaStream_t stream, int a_off = 0, PrepArgs pa = PrepArgs{}) {
    const int e = (d + SLICES - 1) / SLICES;
#define RLIS_SCAN(E) rlis_launch(lightning_scan_kernel<T, E, SILU, VEC, PREP, KCOMP>, grid, THREADS, 0, stream, proj, stride, q_off, k_off, \
                                 v_off, out, state, decay, cu, ctx, slots, nh, d, dv, a_off, pa)
    if (e <= 4) RLIS_SCAN(4);
    else if (e <= 8) RLIS_SCAN(8);
    else if (e <= 16) RLIS_SCAN(16);
    else RLIS_SCAN(32);
#undef RLIS_SCAN
    return RLIS_LAUNCH_CHECK();
}
}  // namespace

extern "C" int rlis_lightning_scan(const void* proj, long long stride, int q_off, int k_off, int v_off, float* out,
                                   float* state, const float* decay, const int* cu_seqlens, const int* ctx_lens,
                                   const int* state_slots, int n_seqs, int nh, int d, int dv, int dtype,
                                   float* activated, int n_tokens, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (d <= 0 || d > SLICES * MAX_E || dv <= 0 || nh <= 0 || nh > 65535) return RLIS_ERR_UNSUPPORTED;
    dim3 grid(n_seqs, nh, (dv + COLS - 1) / COLS);
    if (grid.z > 65535) return RLIS_ERR_UNSUPPORTED;
    if (activated != nullptr) {
        // long steps: silu once into `activated` (float32 [tokens, width], width = the columns up to the end
        // of v, which must start at q_off = 0), then the scan reads that
        const int width = v_off + nh * dv;
        if (q_off != 0 || k_off > v_off || n_tokens <= 0) return RLIS_ERR_UNSUPPORTED;
        const dim3 blocks(n_tokens, (width + 1023) / 1024 < 8 ? (width + 1023) / 1024 : 8);
        if (dtype == RLIS_F32)
            rlis_launch(silu_rows_kernel<float>, blocks, 256, 0, stream, (const float*)proj, stride, activated, width);
        else if (dtype == RLIS_BF16)
            rlis_launch(silu_rows_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)proj, stride, activated, width);
        else
            return RLIS_ERR_UNSUPPORTED;
        return launch_scan<float, false>(activated, (long long)width, q_off, k_off, v_off, out, state, decay, cu_seqlens,
                                         ctx_lens, state_slots, grid, nh, d, dv, stream);
    }
    if (dtype == RLIS_F32)
        return launch_scan<float, true>((const float*)proj, stride, q_off, k_off, v_off, out, state, decay, cu_seqlens,
                                        ctx_lens, state_slots, grid, nh, d, dv, stream);
    if (dtype == RLIS_BF16)
        return launch_scan<bf16, true>((const bf16*)proj, stride, q_off, k_off, v_off, out, state, decay, cu_seqlens,
                                       ctx_lens, state_slots, grid, nh, d, dv, stream);
    return RLIS_ERR_UNSUPPORTED;
}


namespace {
// One row of float32 inputs of a recurrence a token, [q | k | v | a]: nh heads of d (q, k, a) and of dv (v).
//   q: columns q_off of the projection's row, the first rot_dims entries of every head turned with the entries rot_dims
//      / 2 further on by the angle position * inv_freq[i]; q_silu: silu(q) (no rotation then)
//   k: the same rotation, times k_scale; with `lower`: the columns at k_off are the logits z of a forget gate, a = lower +
//      (1 - lower) sigmoid(z + gate_bias) goes to the fourth segment and k = 1 - a
//   v: as projected.
template <typename T>
__global__ __launch_bounds__(256) void recurrence_inputs_kernel(
    const T* __restrict__ proj, long long stride, int q_off, int k_off, int v_off, float* __restrict__ out, int nh, int d,
    int dv, const float* __restrict__ inv_freq, int rot_dims, const int* __restrict__ positions, float k_scale,
    int q_silu, const float* __restrict__ lower, const float* __restrict__ gate_bias, int late_trigger) {
    // Over prompts the walk that follows has few CTAs and wants one to an SM: let in early, while this grid still fills
    // the SMs, its CTAs would land several to an SM wherever room appears first (the walk then runs three times as
    // long).  So in long steps it is let in at the end.
    pdl_wait();
    if (!late_trigger) pdl_trigger();
    const int t = blockIdx.x;
    const int qk = nh * d, hv = nh * dv;
    const int width = 2 * qk + hv + (lower != nullptr ? qk : 0);
    const T* row = proj + (size_t)t * stride;
    float* orow = out + (size_t)t * width;
    const int half = rot_dims >> 1;
    const float pos = rot_dims > 0 ? (float)positions[t] : 0.f;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < 2 * qk + hv; c += gridDim.y * blockDim.x) {
        if (c >= 2 * qk) {
            orow[c] = to_f<T>(row[v_off + c - 2 * qk]);
            continue;
        }
        const bool is_q = c < qk;
        const int hc = is_q ? c : c - qk;                 // head * d + entry
        const T* x = row + (is_q ? q_off : k_off);
        float val = to_f<T>(x[hc]);
        if (!is_q && lower != nullptr) {
            const float l = lower[hc];
            const float z = val + (gate_bias != nullptr ? gate_bias[hc] : 0.f);
            const float a = l + (1.0f - l) * (1.0f / (1.0f + expf(-z)));
            orow[2 * qk + hv + hc] = a;
            orow[c] = 1.0f - a;
            continue;
        }
        const int j = hc % d;
        if (j < rot_dims) {
            const int pj = j < half ? j + half : j - half;
            const float other = to_f<T>(x[hc - j + pj]);
            float sn, cs;
            sincosf(pos * inv_freq[j < half ? j : pj], &sn, &cs);
            val = j < half ? rope_first(val, other, cs, sn) : rope_second(other, val, cs, sn);
        }
        if (is_q && q_silu) val = silu_f(val);
        orow[c] = is_q ? val : val * k_scale;
    }
    if (late_trigger) pdl_trigger();
}
}  // namespace

// out float32 [n_tokens, 2 nh d + nh dv (+ nh d with `lower`)]; inv_freq float32 [rot_dims / 2] and positions int32
// [n_tokens] when rot_dims > 0; lower, gate_bias float32 [nh d] or null.
extern "C" int rlis_recurrence_inputs(const void* proj, long long stride, int q_off, int k_off, int v_off, float* out,
                                      int n_tokens, int nh, int d, int dv, const float* inv_freq, int rot_dims,
                                      const int* positions, float k_scale, int q_silu, const float* lower,
                                      const float* gate_bias, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (nh <= 0 || d <= 0 || dv <= 0 || rot_dims < 0 || rot_dims > d || (rot_dims & 1) ||
        (rot_dims > 0 && (inv_freq == nullptr || positions == nullptr)))
        return RLIS_ERR_UNSUPPORTED;
    const int cols = 2 * nh * d + nh * dv;
    const dim3 blocks(n_tokens, (cols + 1023) / 1024 < 8 ? (cols + 1023) / 1024 : 8);
    const int late = n_tokens >= 64 ? 1 : 0;
    if (dtype == RLIS_F32)
        rlis_launch(recurrence_inputs_kernel<float>, blocks, 256, 0, stream, (const float*)proj, stride, q_off, k_off, v_off,
                    out, nh, d, dv, inv_freq, rot_dims, positions, k_scale, q_silu, lower, gate_bias, late);
    else if (dtype == RLIS_BF16)
        rlis_launch(recurrence_inputs_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)proj, stride, q_off, k_off, v_off,
                    out, nh, d, dv, inv_freq, rot_dims, positions, k_scale, q_silu, lower, gate_bias, late);
    else
        return RLIS_ERR_UNSUPPORTED;
    return RLIS_LAUNCH_CHECK();
}

// The walk over prepared float32 rows [n_tokens, width]: q, k, v at columns q_off, k_off, v_off; a decay a head
// (`decay` float32 [nh]) or, with `decay` null, a decay a token and channel at columns a_off; `key_is_complement`: the
// keys are 1 - decay (what the forget gate's rows hold), and the walk takes them from the decays.
extern "C" int rlis_recurrence_scan(const float* rows, long long width, int q_off, int k_off, int v_off, int a_off,
                                    float* out, float* state, const float* decay, const int* cu_seqlens,
                                    const int* ctx_lens, const int* state_slots, int n_seqs, int nh, int d, int dv,
                                    int key_is_complement, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (d <= 0 || d > SLICES * MAX_E || dv <= 0 || nh <= 0 || nh > 65535) return RLIS_ERR_UNSUPPORTED;
    dim3 grid(n_seqs, nh, (dv + COLS - 1) / COLS);
    if (grid.z > 65535) return RLIS_ERR_UNSUPPORTED;
    if (decay != nullptr)
        return launch_scan<float, false, false>(rows, width, q_off, k_off, v_off, out, state, decay, cu_seqlens, ctx_lens,
                                                state_slots, grid, nh, d, dv, stream);
    if (key_is_complement)      // k = 1 - a: the walk takes it from the decays and does not read the rows' keys
        return launch_scan<float, false, true, 0, true>(rows, width, q_off, k_off, v_off, out, state, nullptr, cu_seqlens,
                                                        ctx_lens, state_slots, grid, nh, d, dv, stream, a_off);
    return launch_scan<float, false, true>(rows, width, q_off, k_off, v_off, out, state, nullptr, cu_seqlens, ctx_lens,
                                           state_slots, grid, nh, d, dv, stream, a_off);
}

// The same walk straight from the projection's rows, its inputs made while the tokens are staged (short steps: every CTA
// of a head makes them again, which a prompt's portion would pay dv / 16 times): rotation of q and k by halves and the
// scale on k with a decay a head (`decay` given), or silu of q and the forget gate with a decay a channel (`lower` given).
extern "C" int rlis_recurrence_scan_rows(const void* proj, long long stride, int q_off, int k_off, int v_off, float* out,
                                         float* state, const float* decay, const int* cu_seqlens, const int* ctx_lens,
                                         const int* state_slots, int n_seqs, int nh, int d, int dv, const float* inv_freq,
                                         int rot_dims, float k_scale, const float* lower, const float* gate_bias, int dtype,
                                         cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (d <= 0 || d > SLICES * MAX_E || dv <= 0 || nh <= 0 || nh > 65535 || (decay == nullptr) == (lower == nullptr))
        return RLIS_ERR_UNSUPPORTED;
    if (rot_dims < 0 || rot_dims > d || (rot_dims & 1) || (rot_dims > 0 && (inv_freq == nullptr || lower != nullptr)))
        return RLIS_ERR_UNSUPPORTED;
    dim3 grid(n_seqs, nh, (dv + COLS - 1) / COLS);
    if (grid.z > 65535) return RLIS_ERR_UNSUPPORTED;
    const PrepArgs pa{inv_freq, rot_dims, k_scale, lower, gate_bias};
#define RLIS_ROWS(T) (decay != nullptr                                                                                         \
        ? launch_scan<T, false, false, 1>((const T*)proj, stride, q_off, k_off, v_off, out, state, decay, cu_seqlens, ctx_lens,   \
                                          state_slots, grid, nh, d, dv, stream, 0, pa)                                            \
        : launch_scan<T, false, true, 2, true>((const T*)proj, stride, q_off, k_off, v_off, out, state, nullptr, cu_seqlens, ctx_lens,  \
                                         state_slots, grid, nh, d, dv, stream, 0, pa))
    if (dtype == RLIS_F32) return RLIS_ROWS(float);
    if (dtype == RLIS_BF16) return RLIS_ROWS(bf16);
#undef RLIS_ROWS
    return RLIS_ERR_UNSUPPORTED;
}

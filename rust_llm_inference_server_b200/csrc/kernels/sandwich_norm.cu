// Norms of blocks that norm a sublayer's result before it joins the residual stream, and plain
// RMSNorms over activations inside a mixer.  All statistics, scales and sums are float32.
//
// post_norm_residual, one CTA a token:
//   y      = sub[t, :] (+ bias)                                   sublayer result, widened
//   resid += mult * scale * (y / sqrt(mean(y^2) + eps) * w_post)  float32, in place (mult a scalar, scale a vector)
//   out    = resid / sqrt(mean(resid^2) + eps) * w_next           rounded once (only if w_next is given)
// so the addition and the norm in front of the next sublayer cost one pass over the row.  With `out` but
// no w_next, out is the stream itself rounded to the activation type (for sublayers that read the stream
// as it is); without `sub` nothing is added and only that copy is made.
//
// sum_norm, one CTA a token, for blocks that norm the sum of the stream and a sublayer's result, and for
// sublayers that are several branches side by side:
//   y     = alpha * resid + ca * N(a; wa) + cb * N(b; wb)          N(x; w) = x / sqrt(mean(x^2) + eps) * w, or x itself
//   y     = y / sqrt(mean(y^2) + eps_out) * w_out                  (only if w_out is given)      when w is null
//   resid = y (float32, in place), out = y rounded to the activation type; every one of resid, a, b, out optional.
//
// act_norm, one CTA a token: out = x / sqrt(mean(x^2) + eps) * w (* sigmoid(gate)), x float32 or the
// activation type with a row stride of its own, gate in the activation type with a row stride.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int THREADS = 256;
constexpr int MAX_PER_THREAD = 32;   // widths up to THREADS * 32 are kept in registers

template <typename T>
__global__ __launch_bounds__(THREADS) void post_norm_residual_kernel(
    const T* __restrict__ sub, const float* __restrict__ bias, const float* __restrict__ w_post,
    const float* __restrict__ scale, float* __restrict__ resid, const float* __restrict__ w_next,
    T* __restrict__ out, int hidden, float eps_post, float eps_next, float mult) {
    pdl_wait_and_trigger();
    __shared__ float scratch[33];
    const size_t base = (size_t)blockIdx.x * hidden;
    float v[MAX_PER_THREAD];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_PER_THREAD; ++i) {
        const int c = threadIdx.x + i * THREADS;
        v[i] = 0.f;
        if (c < hidden && sub != nullptr) {
            v[i] = to_f<T>(sub[base + c]) + (bias != nullptr ? bias[c] : 0.f);
            ss = fmaf(v[i], v[i], ss);
        }
    }
    ss = block_sum(ss, scratch);
    const float r1 = 1.0f / sqrtf(ss / (float)hidden + eps_post);
    float ss2 = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_PER_THREAD; ++i) {
        const int c = threadIdx.x + i * THREADS;
        if (c < hidden) {
            float x = resid[base + c];
            if (sub != nullptr) {
                const float normed = v[i] * r1 * w_post[c];
                x += mult * (scale != nullptr ? scale[c] * normed : normed);
                resid[base + c] = x;
            }
            v[i] = x;
            ss2 = fmaf(x, x, ss2);
        }
    }
    if (w_next == nullptr) {
        if (out != nullptr) {
#pragma unroll
            for (int i = 0; i < MAX_PER_THREAD; ++i) {
                const int c = threadIdx.x + i * THREADS;
                if (c < hidden) out[base + c] = from_f<T>(v[i]);
            }
        }
        return;
    }
    ss2 = block_sum(ss2, scratch);
    const float r2 = 1.0f / sqrtf(ss2 / (float)hidden + eps_next);
#pragma unroll
    for (int i = 0; i < MAX_PER_THREAD; ++i) {
        const int c = threadIdx.x + i * THREADS;
        if (c < hidden) out[base + c] = from_f<T>(v[i] * r2 * w_next[c]);
    }
}

template <typename TIn, typename T>
__global__ __launch_bounds__(THREADS) void act_norm_kernel(
    const TIn* __restrict__ x, long long x_stride, const float* __restrict__ w,
    const T* __restrict__ gate, long long gate_stride, T* __restrict__ out, long long out_stride,
    int width, float eps) {
    pdl_wait_and_trigger();
    __shared__ float scratch[33];
    const TIn* xr = x + (size_t)blockIdx.x * x_stride;
    float v[MAX_PER_THREAD];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_PER_THREAD; ++i) {
        const int c = threadIdx.x + i * THREADS;
        v[i] = 0.f;
        if (c < width) {
            v[i] = to_f<TIn>(xr[c]);
            ss = fmaf(v[i], v[i], ss);
        }
    }
    ss = block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(ss / (float)width + eps);
    T* orow = out + (size_t)blockIdx.x * out_stride;
    const T* grow = gate != nullptr ? gate + (size_t)blockIdx.x * gate_stride : nullptr;
#pragma unroll
    for (int i = 0; i < MAX_PER_THREAD; ++i) {
        const int c = threadIdx.x + i * THREADS;
        if (c < width) {
            float y = v[i] * r * w[c];
            if (grow != nullptr) y *= 1.0f / (1.0f + expf(-to_f<T>(grow[c])));
            orow[c] = from_f<T>(y);
        }
    }
}

// PT = entries of a row that a thread keeps (the width over 256, rounded up to 4, 8 or 32).
template <typename T, int PT>
__global__ __launch_bounds__(THREADS) void sum_norm_kernel(
    const T* __restrict__ a, const float* __restrict__ wa, float ca, const T* __restrict__ b,
    const float* __restrict__ wb, float cb, float* __restrict__ resid, float alpha, const float* __restrict__ w_out,
    T* __restrict__ out, int hidden, float eps_branch, float eps_out) {
    pdl_wait_and_trigger();
    __shared__ float scratch[33];
    const size_t base = (size_t)blockIdx.x * hidden;
    float va[PT], vb[PT];
    float sa = 0.f, sb = 0.f;
#pragma unroll
    for (int i = 0; i < PT; ++i) {
        const int c = threadIdx.x + i * THREADS;
        va[i] = vb[i] = 0.f;
        if (c < hidden) {
            if (a != nullptr) va[i] = to_f<T>(a[base + c]);
            if (b != nullptr) vb[i] = to_f<T>(b[base + c]);
            sa = fmaf(va[i], va[i], sa);
            sb = fmaf(vb[i], vb[i], sb);
        }
    }
    float ra = ca, rb = cb;
    if (a != nullptr && wa != nullptr) ra = ca / sqrtf(block_sum(sa, scratch) / (float)hidden + eps_branch);
    if (b != nullptr && wb != nullptr) rb = cb / sqrtf(block_sum(sb, scratch) / (float)hidden + eps_branch);
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < PT; ++i) {
        const int c = threadIdx.x + i * THREADS;
        if (c < hidden) {
            float y = resid != nullptr ? alpha * resid[base + c] : 0.f;
            if (a != nullptr) y = fmaf(va[i] * ra, wa != nullptr ? wa[c] : 1.0f, y);
            if (b != nullptr) y = fmaf(vb[i] * rb, wb != nullptr ? wb[c] : 1.0f, y);
            va[i] = y;
            ss = fmaf(y, y, ss);
        }
    }
    float r = 1.0f;
    if (w_out != nullptr) r = 1.0f / sqrtf(block_sum(ss, scratch) / (float)hidden + eps_out);
#pragma unroll
    for (int i = 0; i < PT; ++i) {
        const int c = threadIdx.x + i * THREADS;
        if (c < hidden) {
            const float y = w_out != nullptr ? va[i] * r * w_out[c] : va[i];
            if (resid != nullptr) resid[base + c] = y;
            if (out != nullptr) out[base + c] = from_f<T>(y);
        }
    }
}

// out[t, h, :] = x[t, h, :] / sqrt(mean(x[t, h, :]^2) + eps) * w * act(gate[t, h, :]): a norm per head with one
// weight vector for all heads, and a gate (act 0: sigmoid, 1: silu = z sigmoid(z)).  One warp a (token, head).
template <typename T>
__global__ __launch_bounds__(128) void head_norm_gate_kernel(
    const float* __restrict__ x, const float* __restrict__ w, const T* __restrict__ gate, long long gate_stride,
    T* __restrict__ out, int n_units, int nh, int dv, float eps, int act) {
    pdl_wait_and_trigger();
    const int unit = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (unit >= n_units) return;
    const int t = unit / nh, h = unit - t * nh;
    const float* xr = x + (size_t)unit * dv;
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) ss = fmaf(xr[c], xr[c], ss);
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / (float)dv + eps);
    const T* g = gate != nullptr ? gate + (size_t)t * gate_stride + (size_t)h * dv : nullptr;
    T* o = out + (size_t)unit * dv;
    for (int c = lane; c < dv; c += 32) {
        float y = xr[c] * r * (w != nullptr ? w[c] : 1.0f);
        if (g != nullptr) {
            const float z = to_f<T>(g[c]);
            const float sg = 1.0f / (1.0f + expf(-z));
            y *= act == 1 ? z * sg : sg;
        }
        o[c] = from_f<T>(y);
    }
}

// Four consecutive elements as floats (16 bytes of float32, 8 of bfloat16).
template <typename T> struct Quad;
template <> struct Quad<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Quad<bf16> {
    static __device__ __forceinline__ float4 load(const bf16* p) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    static __device__ __forceinline__ void store(bf16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<uint32_t*>(&a);
        raw.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = raw;
    }
};

// The same two kernels for widths that are multiples of 4 on aligned rows: NV vectors of four a thread.
template <typename T, int NV>
__global__ __launch_bounds__(THREADS) void post_norm_residual_vec_kernel(
    const T* __restrict__ sub, const float* __restrict__ bias, const float* __restrict__ w_post,
    const float* __restrict__ scale, float* __restrict__ resid, const float* __restrict__ w_next,
    T* __restrict__ out, int hidden, float eps_post, float eps_next, float mult) {
    pdl_wait_and_trigger();
    __shared__ float scratch[33];
    const size_t base = (size_t)blockIdx.x * hidden;
    float4 v[NV];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = (threadIdx.x + i * THREADS) * 4;
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < hidden && sub != nullptr) {
            v[i] = Quad<T>::load(sub + base + c);
            if (bias != nullptr) {
                const float4 b = Quad<float>::load(bias + c);
                v[i].x += b.x; v[i].y += b.y; v[i].z += b.z; v[i].w += b.w;
            }
            ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss);
            ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
        }
    }
    ss = block_sum(ss, scratch);
    const float r1 = 1.0f / sqrtf(ss / (float)hidden + eps_post);
    float ss2 = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = (threadIdx.x + i * THREADS) * 4;
        if (c < hidden) {
            float4 x = Quad<float>::load(resid + base + c);
            if (sub != nullptr) {
                const float4 w = Quad<float>::load(w_post + c);
                const float4 s = scale != nullptr ? Quad<float>::load(scale + c) : make_float4(1.f, 1.f, 1.f, 1.f);
                const float n0 = v[i].x * r1 * w.x, n1 = v[i].y * r1 * w.y, n2 = v[i].z * r1 * w.z, n3 = v[i].w * r1 * w.w;
                x.x += mult * (scale != nullptr ? s.x * n0 : n0);
                x.y += mult * (scale != nullptr ? s.y * n1 : n1);
                x.z += mult * (scale != nullptr ? s.z * n2 : n2);
                x.w += mult * (scale != nullptr ? s.w * n3 : n3);
                Quad<float>::store(resid + base + c, x);
            }
            v[i] = x;
            ss2 = fmaf(x.x, x.x, ss2); ss2 = fmaf(x.y, x.y, ss2); ss2 = fmaf(x.z, x.z, ss2); ss2 = fmaf(x.w, x.w, ss2);
        }
    }
    if (w_next == nullptr) {
        if (out != nullptr) {
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const int c = (threadIdx.x + i * THREADS) * 4;
                if (c < hidden) Quad<T>::store(out + base + c, v[i]);
            }
        }
        return;
    }
    ss2 = block_sum(ss2, scratch);
    const float r2 = 1.0f / sqrtf(ss2 / (float)hidden + eps_next);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = (threadIdx.x + i * THREADS) * 4;
        if (c < hidden) {
            const float4 w = Quad<float>::load(w_next + c);
            Quad<T>::store(out + base + c, make_float4(v[i].x * r2 * w.x, v[i].y * r2 * w.y, v[i].z * r2 * w.z, v[i].w * r2 * w.w));
        }
    }
}

template <typename TIn, typename T, int NV>
__global__ __launch_bounds__(THREADS) void act_norm_vec_kernel(
    const TIn* __restrict__ x, long long x_stride, const float* __restrict__ w,
    const T* __restrict__ gate, long long gate_stride, T* __restrict__ out, long long out_stride,
    int width, float eps) {
    pdl_wait_and_trigger();
    __shared__ float scratch[33];
    const TIn* xr = x + (size_t)blockIdx.x * x_stride;
    float4 v[NV];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = (threadIdx.x + i * THREADS) * 4;
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < width) {
            v[i] = Quad<TIn>::load(xr + c);
            ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss);
            ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
        }
    }
    ss = block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(ss / (float)width + eps);
    T* orow = out + (size_t)blockIdx.x * out_stride;
    const T* grow = gate != nullptr ? gate + (size_t)blockIdx.x * gate_stride : nullptr;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = (threadIdx.x + i * THREADS) * 4;
        if (c < width) {
            const float4 ww = Quad<float>::load(w + c);
            float4 y = make_float4(v[i].x * r * ww.x, v[i].y * r * ww.y, v[i].z * r * ww.z, v[i].w * r * ww.w);
            if (grow != nullptr) {
                const float4 gt = Quad<T>::load(grow + c);
                y.x *= 1.0f / (1.0f + expf(-gt.x)); y.y *= 1.0f / (1.0f + expf(-gt.y));
                y.z *= 1.0f / (1.0f + expf(-gt.z)); y.w *= 1.0f / (1.0f + expf(-gt.w));
            }
            Quad<T>::store(orow + c, y);
        }
    }
}

template <typename T>
__global__ void bias_act_vec_kernel(const T* __restrict__ x, const float* __restrict__ b, T* __restrict__ out,
                                    long long n4, int width, int act) {
    pdl_wait_and_trigger();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
        float4 v = Quad<T>::load(x + i * 4);
        if (b != nullptr) {
            const float4 bb = Quad<float>::load(b + (i * 4) % width);
            v.x += bb.x; v.y += bb.y; v.z += bb.z; v.w += bb.w;
        }
        if (act == 1) {
            v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f); v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f);
            v.x *= v.x; v.y *= v.y; v.z *= v.z; v.w *= v.w;
        }
        Quad<T>::store(out + i * 4, v);
    }
}

template <typename T>
static bool aligned_for_quads(const void* p) { return ((uintptr_t)p) % (4 * sizeof(T)) == 0; }

// out = act(x + b): act 0 none, 1 the square of max(., 0).  Element-wise, float32 inside.
template <typename T>
__global__ void bias_act_kernel(const T* __restrict__ x, const float* __restrict__ b, T* __restrict__ out,
                                long long n, int width, int act) {
    pdl_wait_and_trigger();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        float v = to_f<T>(x[i]) + (b != nullptr ? b[i % width] : 0.f);
        if (act == 1) {
            v = fmaxf(v, 0.f);
            v = v * v;
        }
        out[i] = from_f<T>(v);
    }
}
}  // namespace

extern "C" int rlis_post_norm_residual(const void* sub, const float* bias, const float* w_post, const float* scale,
                                       float* resid, const float* w_next, void* out, int n_tokens, int hidden,
                                       float eps_post, float eps_next, float mult, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (hidden <= 0 || hidden > THREADS * MAX_PER_THREAD) return RLIS_ERR_UNSUPPORTED;
    if (hidden % 4 == 0 && (dtype == RLIS_F32 || dtype == RLIS_BF16)) {
        const int nv = (hidden / 4 + THREADS - 1) / THREADS;
#define RLIS_PNR(T, NV) rlis_launch(post_norm_residual_vec_kernel<T, NV>, n_tokens, THREADS, 0, stream, (const T*)sub, bias, \
                                    w_post, scale, resid, w_next, (T*)out, hidden, eps_post, eps_next, mult)
#define RLIS_PNR_T(T) do { if (nv <= 1) RLIS_PNR(T, 1); else if (nv <= 2) RLIS_PNR(T, 2); else if (nv <= 4) RLIS_PNR(T, 4); \
                           else RLIS_PNR(T, 8); } while (0)
        if (dtype == RLIS_F32) RLIS_PNR_T(float); else RLIS_PNR_T(bf16);
#undef RLIS_PNR_T
#undef RLIS_PNR
        return RLIS_LAUNCH_CHECK();
    }
    if (dtype == RLIS_F32)
        rlis_launch(post_norm_residual_kernel<float>, n_tokens, THREADS, 0, stream, (const float*)sub, bias, w_post,
                    scale, resid, w_next, (float*)out, hidden, eps_post, eps_next, mult);
    else if (dtype == RLIS_BF16)
        rlis_launch(post_norm_residual_kernel<bf16>, n_tokens, THREADS, 0, stream, (const bf16*)sub, bias, w_post,
                    scale, resid, w_next, (bf16*)out, hidden, eps_post, eps_next, mult);
    else
        return RLIS_ERR_UNSUPPORTED;
    return RLIS_LAUNCH_CHECK();
}

// x_f32 != 0: x is float32 whatever `dtype` (the activation type of gate and out) says.
extern "C" int rlis_act_norm(const void* x, long long x_stride, int x_f32, const float* w, const void* gate,
                             long long gate_stride, void* out, long long out_stride, int n_tokens, int width,
                             float eps, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (width <= 0 || width > THREADS * MAX_PER_THREAD) return RLIS_ERR_UNSUPPORTED;
    const bool in32 = dtype == RLIS_F32 || x_f32;
    const bool quads = width % 4 == 0 && x_stride % 4 == 0 && gate_stride % 4 == 0 && out_stride % 4 == 0 &&
                       (in32 ? aligned_for_quads<float>(x) : aligned_for_quads<bf16>(x)) &&
                       (dtype == RLIS_F32 ? aligned_for_quads<float>(out) && aligned_for_quads<float>(gate)
                                          : aligned_for_quads<bf16>(out) && aligned_for_quads<bf16>(gate));
    if (quads && (dtype == RLIS_F32 || dtype == RLIS_BF16)) {
        const int nv = (width / 4 + THREADS - 1) / THREADS;
#define RLIS_AN(TI, T, NV) rlis_launch(act_norm_vec_kernel<TI, T, NV>, n_tokens, THREADS, 0, stream, (const TI*)x, x_stride, w, \
                                       (const T*)gate, gate_stride, (T*)out, out_stride, width, eps)
#define RLIS_AN_T(TI, T) do { if (nv <= 1) RLIS_AN(TI, T, 1); else if (nv <= 2) RLIS_AN(TI, T, 2); else if (nv <= 4) RLIS_AN(TI, T, 4); \
                              else RLIS_AN(TI, T, 8); } while (0)
        if (dtype == RLIS_F32) RLIS_AN_T(float, float);
        else if (x_f32) RLIS_AN_T(float, bf16);
        else RLIS_AN_T(bf16, bf16);
#undef RLIS_AN_T
#undef RLIS_AN
        return RLIS_LAUNCH_CHECK();
    }
    if (dtype == RLIS_F32)
        rlis_launch(act_norm_kernel<float, float>, n_tokens, THREADS, 0, stream, (const float*)x, x_stride, w,
                    (const float*)gate, gate_stride, (float*)out, out_stride, width, eps);
    else if (dtype == RLIS_BF16 && x_f32)
        rlis_launch(act_norm_kernel<float, bf16>, n_tokens, THREADS, 0, stream, (const float*)x, x_stride, w,
                    (const bf16*)gate, gate_stride, (bf16*)out, out_stride, width, eps);
    else if (dtype == RLIS_BF16)
        rlis_launch(act_norm_kernel<bf16, bf16>, n_tokens, THREADS, 0, stream, (const bf16*)x, x_stride, w,
                    (const bf16*)gate, gate_stride, (bf16*)out, out_stride, width, eps);
    else
        return RLIS_ERR_UNSUPPORTED;
    return RLIS_LAUNCH_CHECK();
}

extern "C" int rlis_bias_act(const void* x, const float* b, void* out, long long n_rows, int width, int act,
                             int dtype, cudaStream_t stream) {
    const long long n = n_rows * width;
    if (n <= 0) return 0;
    if (act < 0 || act > 1) return RLIS_ERR_UNSUPPORTED;
    if (width % 4 == 0 && (dtype == RLIS_F32 || dtype == RLIS_BF16)) {
        const long long n4 = n / 4;
        const unsigned vblocks = (unsigned)((n4 + 255) / 256 < 8192 ? (n4 + 255) / 256 : 8192);
        if (dtype == RLIS_F32)
            rlis_launch(bias_act_vec_kernel<float>, vblocks, 256, 0, stream, (const float*)x, b, (float*)out, n4, width, act);
        else
            rlis_launch(bias_act_vec_kernel<bf16>, vblocks, 256, 0, stream, (const bf16*)x, b, (bf16*)out, n4, width, act);
        return RLIS_LAUNCH_CHECK();
    }
    const unsigned blocks = (unsigned)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
    if (dtype == RLIS_F32)
        rlis_launch(bias_act_kernel<float>, blocks, 256, 0, stream, (const float*)x, b, (float*)out, n, width, act);
    else if (dtype == RLIS_BF16)
        rlis_launch(bias_act_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)x, b, (bf16*)out, n, width, act);
    else
        return RLIS_ERR_UNSUPPORTED;
    return RLIS_LAUNCH_CHECK();
}

// a, b: sublayer results [T, hidden] in the activation type (null: none); wa, wb: their norms' weights (null: the
// result joins as it is); resid float32 [T, hidden] (null: no stream term, nothing written back); w_out null: no
// norm of the sum; out null: no rounded copy.
extern "C" int rlis_sum_norm(const void* a, const float* wa, float ca, const void* b, const float* wb, float cb,
                             float* resid, float alpha, const float* w_out, void* out, int n_tokens, int hidden,
                             float eps_branch, float eps_out, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (hidden <= 0 || hidden > THREADS * MAX_PER_THREAD || (resid == nullptr && out == nullptr)) return RLIS_ERR_UNSUPPORTED;
#define RLIS_SUM_NORM(T, PT)                                                                                       \
    rlis_launch(sum_norm_kernel<T, PT>, n_tokens, THREADS, 0, stream, (const T*)a, wa, ca, (const T*)b, wb, cb, resid, \
                alpha, w_out, (T*)out, hidden, eps_branch, eps_out)
#define RLIS_SUM_NORM_T(T)                                                                                         \
    do {                                                                                                           \
        if (hidden <= THREADS * 4) RLIS_SUM_NORM(T, 4);                                                            \
        else if (hidden <= THREADS * 8) RLIS_SUM_NORM(T, 8);                                                       \
        else RLIS_SUM_NORM(T, MAX_PER_THREAD);                                                                     \
    } while (0)
    if (dtype == RLIS_F32) RLIS_SUM_NORM_T(float);
    else if (dtype == RLIS_BF16) RLIS_SUM_NORM_T(bf16);
    else return RLIS_ERR_UNSUPPORTED;
#undef RLIS_SUM_NORM_T
#undef RLIS_SUM_NORM
    return RLIS_LAUNCH_CHECK();
}

// x float32 [T, nh, dv] contiguous; w float32 [dv]; gate (null: none) in the activation type, head h of token t
// at gate + t * gate_stride + h * dv; out [T, nh, dv] in the activation type.
extern "C" int rlis_head_norm_gate(const float* x, const float* w, const void* gate, long long gate_stride, void* out,
                                   int n_tokens, int nh, int dv, float eps, int act, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const long long units = (long long)n_tokens * nh;
    if (nh <= 0 || dv <= 0 || units > 0x7fffffffLL || act < 0 || act > 1) return RLIS_ERR_UNSUPPORTED;
    const unsigned blocks = (unsigned)((units + 3) / 4);
    if (dtype == RLIS_F32)
        rlis_launch(head_norm_gate_kernel<float>, blocks, 128, 0, stream, x, w, (const float*)gate, gate_stride, (float*)out,
                    (int)units, nh, dv, eps, act);
    else if (dtype == RLIS_BF16)
        rlis_launch(head_norm_gate_kernel<bf16>, blocks, 128, 0, stream, x, w, (const bf16*)gate, gate_stride, (bf16*)out,
                    (int)units, nh, dv, eps, act);
    else
        return RLIS_ERR_UNSUPPORTED;
    return RLIS_LAUNCH_CHECK();
}

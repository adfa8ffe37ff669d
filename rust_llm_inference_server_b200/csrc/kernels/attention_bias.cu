// Causal grouped-query attention with per-head RMS-normed queries and keys, a learned bias by
// distance, values of their own width, optional mixing of a layer's values with another layer's,
// and a gate on every head's output.  No rotation: positions enter through the bias alone.
//
//   q_h = rmsnorm(q_h) * wq,  k_g = rmsnorm(k_g) * wk              (weights shared by the heads)
//   v_g = (1 - lambda) v_g + lambda v_other_g                      (where a layer mixes; that is what is cached)
//   score(i, j) = scale * q_h(i) . k_g(j) + bias[min(i - j, n_dist - 1), h],  j <= i (and i - j < window)
//   out_h(i) = sigmoid(gate_h(i)) * sum_j softmax_j(score) v_g(j)
//
// Options that other designs use, each off unless its argument is given: the first `rot_dims` entries of every
// query and key head are rotated before the norm, entry 2i with entry 2i+1 by the angle position * inv_freq[i]
// (cos and sin times `rot_mag`); queries are multiplied, after their norm, by 1 + coef * ln(floor((p + 1) /
// every) + 1) at position p; slope_h * (i - j) is subtracted from a score; exp(sink_h) joins the softmax's
// denominator (a term without key or value).  Values that are the keys as projected are had by v_off = k_off.
// `rot_half`: the rotation pairs entry i with entry i + rot_dims / 2 instead (the pair (a, b) becomes (a cos - b sin,
// b cos + a sin) either way).  `proj_bias` (float32, one entry a column of the projection's row): added to queries,
// keys and values as they are read.  `gate_cols` > 1: the gate has one logit a channel of every head (gate[t, h *
// dv + c]) instead of one a head.
//
// `bias` is a float32 table [n_dist, n_heads] by distance (the host turns bucket rules into it; all
// distances from n_dist - 1 on share the last row).  Norms, scores, softmax, value sums, the mixing and
// the gate are float32 whatever the element type.
//
// norm_store: one warp per (token, query or key/value head); writes normed queries to q_out and
// normed keys and (mixed) values into the paged cache [page, kv head, slot in page, d | dv].
// attention: one warp per (token, query head), keys in blocks of 32 that start at multiples of 32, so
// the order of every sum depends on the query's position only.  The kernel of the float32 path and
// the fallback of the bfloat16 path for sizes the tensor-core kernels refuse.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int WARPS = 4;
constexpr int MAX_D = 256;     // head sizes up to 256 (8 entries a lane)

template <typename T>
__global__ __launch_bounds__(WARPS * 32) void qk_norm_store_kernel(
    const T* __restrict__ proj, long long stride, int q_off, int k_off, int v_off,
    const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
    const T* __restrict__ v_other, long long v_other_stride, float lambda,
    T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache, const int* __restrict__ slots,
    int n_units, int nh, int nkv, int d, int dv, int page_size,
    const float* __restrict__ inv_freq, int rot_dims, float rot_mag, const int* __restrict__ positions,
    float q_temp_coef, int q_temp_every, int rot_half, const float* __restrict__ proj_bias) {
    pdl_wait_and_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int unit = blockIdx.x * WARPS + warp;
    if (unit >= n_units) return;
    const int per = nh + nkv;
    const int t = unit / per, u = unit - t * per;
    const T* row = proj + (size_t)t * stride;
    const bool is_q = u < nh;
    const int x_col = is_q ? q_off + u * d : k_off + (u - nh) * d;
    const T* x = row + x_col;
    const float* xb = proj_bias != nullptr ? proj_bias + x_col : nullptr;
    const float* w = is_q ? q_w : k_w;
    float v[MAX_D / 32];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) {
        const int c = lane + 32 * i;
        v[i] = c < d ? to_f<T>(x[c]) + (xb != nullptr ? xb[c] : 0.f) : 0.f;
    }
    const int pos = positions != nullptr ? positions[t] : 0;
    if (rot_dims > 0 && rot_half) {
        // entry c turns with entry c +- rot_dims / 2, read again from the row
        const int half = rot_dims >> 1;
#pragma unroll
        for (int i = 0; i < MAX_D / 32; ++i) {
            const int c = lane + 32 * i;
            if (c < rot_dims) {
                const int pc = c < half ? c + half : c - half;
                const float other = to_f<T>(x[pc]) + (xb != nullptr ? xb[pc] : 0.f);
                float sn, cs;
                sincosf((float)pos * inv_freq[c < half ? c : pc], &sn, &cs);
                sn *= rot_mag;
                cs *= rot_mag;
                v[i] = c < half ? rope_first(v[i], other, cs, sn) : rope_second(other, v[i], cs, sn);
            }
        }
    } else if (rot_dims > 0) {
        // lanes 2j and 2j+1 hold a pair (32 i is even)
#pragma unroll
        for (int i = 0; i < MAX_D / 32; ++i) {
            const int c = lane + 32 * i;
            const float other = __shfl_xor_sync(0xffffffffu, v[i], 1);
            if (c < rot_dims) {
                float sn, cs;
                sincosf((float)pos * inv_freq[c >> 1], &sn, &cs);
                sn *= rot_mag;
                cs *= rot_mag;
                v[i] = (c & 1) ? rope_second(other, v[i], cs, sn) : rope_first(v[i], other, cs, sn);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) ss = fmaf(v[i], v[i], ss);
    ss = warp_sum(ss);
    float r = w != nullptr ? 1.0f / sqrtf(ss / (float)d + eps) : 1.0f;
    const bool scaled = w != nullptr || (is_q && q_temp_every > 0);
    if (is_q && q_temp_every > 0) r *= 1.0f + q_temp_coef * logf((float)((pos + 1) / q_temp_every + 1));
    T* dst = nullptr;
    long long vrow = -1;
    if (is_q) {
        dst = q_out + ((size_t)t * nh + u) * d;
    } else {
        const int slot = slots != nullptr ? slots[t] : -1;
        if (slot >= 0) {
            const long long page = slot / page_size;
            const int off = slot % page_size;
            const long long r0 = (page * nkv + (u - nh)) * page_size + off;
            dst = k_cache + r0 * d;
            vrow = r0 * dv;
        }
    }
    if (dst != nullptr) {
#pragma unroll
        for (int i = 0; i < MAX_D / 32; ++i) {
            const int c = lane + 32 * i;
            if (c < d) dst[c] = from_f<T>(scaled ? v[i] * r * (w != nullptr ? w[c] : 1.0f) : v[i]);
        }
    }
    if (vrow >= 0) {
        const int g = u - nh;
        const T* vs = row + v_off + g * dv;
        const float* vb = proj_bias != nullptr ? proj_bias + v_off + g * dv : nullptr;
        const T* vo = v_other != nullptr ? v_other + (size_t)t * v_other_stride + g * dv : nullptr;
        for (int c = lane; c < dv; c += 32) {
            float val = to_f<T>(vs[c]) + (vb != nullptr ? vb[c] : 0.f);
            if (vo != nullptr) val = (1.0f - lambda) * val + lambda * to_f<T>(vo[c]);
            v_cache[vrow + c] = from_f<T>(val);
        }
    }
}

// The same with 16-byte loads and stores: d / VN lanes a (token, head) (VN elements a vector: 8 of bfloat16, 4
// of float32), so a warp takes 32 VN / d of them; for head sizes d = VN * 2^k up to 32 VN, value widths that
// are multiples of VN, and rows, offsets and pointers on 16-byte boundaries.
template <typename T>
__global__ __launch_bounds__(WARPS * 32) void qk_norm_store_vec_kernel(
    const T* __restrict__ proj, long long stride, int q_off, int k_off, int v_off,
    const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
    const T* __restrict__ v_other, long long v_other_stride, float lambda,
    T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache, const int* __restrict__ slots,
    int n_units, int nh, int nkv, int d, int dv, int page_size, int lanes,
    const float* __restrict__ inv_freq, int rot_dims, float rot_mag, const int* __restrict__ positions,
    float q_temp_coef, int q_temp_every, int rot_half, const float* __restrict__ proj_bias) {
    pdl_wait_and_trigger();
    constexpr int VN = Vec16<T>::N;
    const int lane = threadIdx.x & 31;
    const int sub = lane / lanes, li = lane - sub * lanes;          // which of the warp's units, and the lane in it
    const int per_warp = 32 / lanes;
    const int unit = (blockIdx.x * WARPS + (threadIdx.x >> 5)) * per_warp + sub;
    const bool live = unit < n_units;
    const int per = nh + nkv;
    const int t = live ? unit / per : 0, u = live ? unit - t * per : 0;
    const T* row = proj + (size_t)t * stride;
    const bool is_q = u < nh;
    const int x_col = is_q ? q_off + u * d : k_off + (u - nh) * d;
    const T* x = row + x_col;
    const float* xb = proj_bias != nullptr ? proj_bias + x_col : nullptr;
    const float* w = is_q ? q_w : k_w;
    float v[VN];
    load16<T>(x + li * VN, v);
    if (xb != nullptr) {
#pragma unroll
        for (int i = 0; i < VN; ++i) v[i] += xb[li * VN + i];
    }
    const int pos = positions != nullptr ? positions[t] : 0;
    if (rot_dims > 0 && rot_half) {
        // a lane's VN entries lie in one half of the rotated part (rot_dims / 2 is a multiple of VN): their
        // partners are the VN entries rot_dims / 2 further on or back, read again from the row
        const int half = rot_dims >> 1, c0 = li * VN;
        if (c0 < rot_dims) {
            const int p0 = c0 < half ? c0 + half : c0 - half;
            float o[VN];
            load16<T>(x + p0, o);
#pragma unroll
            for (int i = 0; i < VN; ++i) {
                if (xb != nullptr) o[i] += xb[p0 + i];
                float sn, cs;
                sincosf((float)pos * inv_freq[(c0 < half ? c0 : p0) + i], &sn, &cs);
                sn *= rot_mag;
                cs *= rot_mag;
                v[i] = c0 < half ? rope_first(v[i], o[i], cs, sn) : rope_second(o[i], v[i], cs, sn);
            }
        }
    } else if (rot_dims > 0) {
        // a lane's VN entries are whole pairs
#pragma unroll
        for (int i = 0; i < VN; i += 2) {
            const int c = li * VN + i;
            if (c < rot_dims) {
                float sn, cs;
                sincosf((float)pos * inv_freq[c >> 1], &sn, &cs);
                sn *= rot_mag;
                cs *= rot_mag;
                const float a = v[i], b = v[i + 1];
                v[i] = rope_first(a, b, cs, sn);
                v[i + 1] = rope_second(a, b, cs, sn);
            }
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VN; ++i) ss = fmaf(v[i], v[i], ss);
    for (int o = lanes >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);     // within the unit's lanes
    if (!live) return;
    float r = w != nullptr ? 1.0f / sqrtf(ss / (float)d + eps) : 1.0f;
    const bool scaled = w != nullptr || (is_q && q_temp_every > 0);
    if (is_q && q_temp_every > 0) r *= 1.0f + q_temp_coef * logf((float)((pos + 1) / q_temp_every + 1));
    T* dst = nullptr;
    long long vrow = -1;
    if (is_q) {
        dst = q_out + ((size_t)t * nh + u) * d;
    } else {
        const int slot = slots != nullptr ? slots[t] : -1;
        if (slot >= 0) {
            const long long r0 = ((long long)(slot / page_size) * nkv + (u - nh)) * page_size + slot % page_size;
            dst = k_cache + r0 * d;
            vrow = r0 * dv;
        }
    }
    if (dst != nullptr) {
        alignas(16) T o[VN];
#pragma unroll
        for (int i = 0; i < VN; ++i) o[i] = from_f<T>(scaled ? v[i] * r * (w != nullptr ? w[li * VN + i] : 1.0f) : v[i]);
        *reinterpret_cast<uint4*>(dst + li * VN) = *reinterpret_cast<const uint4*>(o);
    }
    if (vrow >= 0) {
        const int g = u - nh;
        const T* vs = row + v_off + g * dv;
        const T* vo = v_other != nullptr ? v_other + (size_t)t * v_other_stride + g * dv : nullptr;
        for (int c = li * VN; c < dv; c += lanes * VN) {
            float a[VN];
            load16<T>(vs + c, a);
            if (proj_bias != nullptr) {
#pragma unroll
                for (int i = 0; i < VN; ++i) a[i] += proj_bias[v_off + g * dv + c + i];
            }
            if (vo != nullptr) {
                float b[VN];
                load16<T>(vo + c, b);
#pragma unroll
                for (int i = 0; i < VN; ++i) a[i] = (1.0f - lambda) * a[i] + lambda * b[i];
            }
            alignas(16) T o[VN];
#pragma unroll
            for (int i = 0; i < VN; ++i) o[i] = from_f<T>(a[i]);
            *reinterpret_cast<uint4*>(v_cache + vrow + c) = *reinterpret_cast<const uint4*>(o);
        }
    }
}

template <typename T>
__global__ __launch_bounds__(WARPS * 32) void attn_bias_kernel(
    const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache, T* __restrict__ out,
    const float* __restrict__ bias, int n_dist, const T* __restrict__ gate, long long gate_stride,
    const int* __restrict__ seq_of_token, const int* __restrict__ positions, const int* __restrict__ block_tables,
    const int* __restrict__ token_rows, int max_blocks, int n_rows, int nh, int nkv, int d, int dv, int page_size,
    float scale, int window, const float* __restrict__ sinks, const float* __restrict__ slopes, int gate_cols) {
    pdl_wait();
    extern __shared__ float qs_all[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gw = blockIdx.x * WARPS + warp;
    if (gw >= n_rows) return;  // no block-wide barrier below
    const int ti = gw / nh, h = gw - ti * nh;
    const int t = token_rows != nullptr ? token_rows[ti] : ti;
    const int kvh = h / (nh / nkv);
    const int pos = positions[t];
    const int* table = block_tables + (size_t)seq_of_token[t] * max_blocks;
    float* qs = qs_all + warp * d;
    const T* qrow = q + ((size_t)t * nh + h) * d;
    for (int j = lane; j < d; j += 32) qs[j] = to_f<T>(qrow[j]);
    __syncwarp();

    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const float slope = slopes != nullptr ? slopes[h] : 0.f;
    float m = -INFINITY, l = 0.f;
    float acc[MAX_D / 32];
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) acc[i] = 0.f;

    for (int kb = lo - (lo & 31); kb <= pos; kb += 32) {
        const int key = kb + lane;
        const bool valid = key >= lo && key <= pos;
        float s = -INFINITY;
        long long row = -1;      // row of this lane's key in the pools, or -1: hidden, or a page the host did not map
        if (valid) {
            const int page = table[key / page_size];
            if (page < 0) {
                s = NAN;
            } else {
                row = ((long long)page * nkv + kvh) * page_size + key % page_size;
                const T* krow = k_cache + row * d;
                float dot = 0.f;
                for (int j = 0; j < d; ++j) dot = fmaf(qs[j], to_f<T>(krow[j]), dot);
                s = dot * scale;
                if (bias != nullptr) s += bias[(size_t)min(pos - key, n_dist - 1) * nh + h];
                if (slopes != nullptr) s -= slope * (float)(pos - key);
            }
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = valid ? expf(s - m_new) : 0.f;
        const float corr = expf(m - m_new);
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < MAX_D / 32; ++i) acc[i] *= corr;
#pragma unroll 8
        for (int kk = 0; kk < 32; ++kk) {
            const float pk = __shfl_sync(0xffffffffu, p, kk);
            const long long r = __shfl_sync(0xffffffffu, row, kk);
            const bool use = pk != 0.f && r >= 0;  // uniform over the warp
            const T* vrow = v_cache + (use ? r * dv : 0);
#pragma unroll
            for (int i = 0; i < MAX_D / 32; ++i) {
                const int c = lane + 32 * i;
                if (c < dv) {
                    const float v = to_f<T>(vrow[c]);
                    acc[i] = use ? fmaf(pk, v, acc[i]) : acc[i];
                }
            }
        }
        m = m_new;
    }
    if (sinks != nullptr) {
        // one more term of the denominator, without a key or a value
        const float sk = sinks[h];
        const float m_new = fmaxf(m, sk);
        const float corr = expf(m - m_new);
        l = l * corr + expf(sk - m_new);
#pragma unroll
        for (int i = 0; i < MAX_D / 32; ++i) acc[i] *= corr;
    }
    float g = 1.0f;
    const bool by_channel = gate != nullptr && gate_cols > 1;
    if (gate != nullptr && !by_channel) g = 1.0f / (1.0f + expf(-to_f<T>(gate[(size_t)t * gate_stride + h])));
    T* orow = out + ((size_t)t * nh + h) * dv;
    const float inv_l = g / l;
    const T* grow = by_channel ? gate + (size_t)t * gate_stride + (size_t)h * dv : nullptr;
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) {
        const int c = lane + 32 * i;
        if (c < dv) {
            float y = acc[i] * inv_l;
            if (by_channel) y *= 1.0f / (1.0f + expf(-to_f<T>(grow[c])));
            orow[c] = from_f<T>(y);
        }
    }
    pdl_trigger();
}
}  // namespace

// proj [T, stride]: the stacked projection's rows; queries at column q_off (nh heads of d), keys at
// k_off (nkv of d), values at v_off (nkv of dv).  q_w, k_w float32 [d] (null: no norm).  v_other (null:
// no mixing): rows of another layer's values [T, v_other_stride], mixed in with weight lambda.
// slots null: nothing is stored (the call reads another call's cache) and only q_out is made.
extern "C" int rlis_qk_norm_store(const void* proj, long long stride, int q_off, int k_off, int v_off,
                                  const float* q_w, const float* k_w, float eps, const void* v_other,
                                  long long v_other_stride, float lambda, void* q_out, void* k_cache, void* v_cache,
                                  const int* slots, int n_tokens, int nh, int nkv, int d, int dv, int page_size,
                                  const float* inv_freq, int rot_dims, float rot_mag, const int* positions,
                                  float q_temp_coef, int q_temp_every, int rot_half, const float* proj_bias, int dtype,
                                  cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (d <= 0 || d > MAX_D || dv <= 0 || nh <= 0 || nkv <= 0) return RLIS_ERR_UNSUPPORTED;
    if (rot_dims < 0 || rot_dims > d || (rot_dims & 1) || (rot_dims > 0 && (inv_freq == nullptr || positions == nullptr)) ||
        (q_temp_every > 0 && positions == nullptr))
        return RLIS_ERR_UNSUPPORTED;
    const long long units = (long long)n_tokens * (nh + nkv);
    if (units > 0x7fffffffLL) return RLIS_ERR_UNSUPPORTED;
    {
        // the vector form where everything lies on 16-byte boundaries and a head is VN * 2^k elements
        const int vn = dtype == RLIS_F32 ? 4 : 8;
        const int lanes = d / vn;
        const uintptr_t ptrs = reinterpret_cast<uintptr_t>(proj) | reinterpret_cast<uintptr_t>(v_other) |
                               reinterpret_cast<uintptr_t>(q_out) | reinterpret_cast<uintptr_t>(k_cache) |
                               reinterpret_cast<uintptr_t>(v_cache);
        const bool vec = (dtype == RLIS_F32 || dtype == RLIS_BF16) && d % vn == 0 && dv % vn == 0 && lanes >= 1 &&
                         lanes <= 32 && (lanes & (lanes - 1)) == 0 && (ptrs & 15) == 0 && stride % vn == 0 &&
                         v_other_stride % vn == 0 && q_off % vn == 0 && k_off % vn == 0 && v_off % vn == 0 &&
                         (!rot_half || rot_dims == 0 || (rot_dims / 2) % vn == 0);
        if (vec) {
            const int per_warp = 32 / lanes;
            const unsigned vblocks = (unsigned)((units + (long long)WARPS * per_warp - 1) / (WARPS * per_warp));
            if (dtype == RLIS_F32)
                rlis_launch(qk_norm_store_vec_kernel<float>, vblocks, WARPS * 32, 0, stream, (const float*)proj, stride, q_off,
                            k_off, v_off, q_w, k_w, eps, (const float*)v_other, v_other_stride, lambda, (float*)q_out,
                            (float*)k_cache, (float*)v_cache, slots, (int)units, nh, nkv, d, dv, page_size, lanes, inv_freq, rot_dims,
                            rot_mag, positions, q_temp_coef, q_temp_every, rot_half, proj_bias);
            else
                rlis_launch(qk_norm_store_vec_kernel<bf16>, vblocks, WARPS * 32, 0, stream, (const bf16*)proj, stride, q_off,
                            k_off, v_off, q_w, k_w, eps, (const bf16*)v_other, v_other_stride, lambda, (bf16*)q_out,
                            (bf16*)k_cache, (bf16*)v_cache, slots, (int)units, nh, nkv, d, dv, page_size, lanes, inv_freq, rot_dims,
                            rot_mag, positions, q_temp_coef, q_temp_every, rot_half, proj_bias);
            return RLIS_LAUNCH_CHECK();
        }
    }
    const unsigned blocks = (unsigned)((units + WARPS - 1) / WARPS);
    if (dtype == RLIS_F32)
        rlis_launch(qk_norm_store_kernel<float>, blocks, WARPS * 32, 0, stream, (const float*)proj, stride, q_off, k_off,
                    v_off, q_w, k_w, eps, (const float*)v_other, v_other_stride, lambda, (float*)q_out, (float*)k_cache,
                    (float*)v_cache, slots, (int)units, nh, nkv, d, dv, page_size, inv_freq, rot_dims, rot_mag, positions,
                    q_temp_coef, q_temp_every, rot_half, proj_bias);
    else if (dtype == RLIS_BF16)
        rlis_launch(qk_norm_store_kernel<bf16>, blocks, WARPS * 32, 0, stream, (const bf16*)proj, stride, q_off, k_off,
                    v_off, q_w, k_w, eps, (const bf16*)v_other, v_other_stride, lambda, (bf16*)q_out, (bf16*)k_cache,
                    (bf16*)v_cache, slots, (int)units, nh, nkv, d, dv, page_size, inv_freq, rot_dims, rot_mag, positions,
                    q_temp_coef, q_temp_every, rot_half, proj_bias);
    else
        return RLIS_ERR_UNSUPPORTED;
    return RLIS_LAUNCH_CHECK();
}

// q [T, nh d]; k_cache [pages, nkv, page_size, d]; v_cache [pages, nkv, page_size, dv]; out [T, nh dv];
// bias float32 [n_dist, nh] or null; gate (null: none): logits, head h of token t at gate[t * gate_stride + h];
// sinks, slopes float32 [nh] or null.  gate_cols dv: the gate has a logit a channel, gate[t * gate_stride + h * dv + c].
extern "C" int rlis_attention_bias(const void* q, const void* k_cache, const void* v_cache, void* out,
                                   const float* bias, int n_dist, const void* gate, long long gate_stride,
                                   const int* seq_of_token, const int* positions, const int* block_tables,
                                   const int* token_rows, int max_blocks, int n_tokens, int nh, int nkv, int d, int dv,
                                   int page_size, float scale, int window, const float* sinks, const float* slopes,
                                   int gate_cols, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (d <= 0 || d > MAX_D || dv <= 0 || dv > MAX_D || nkv <= 0 || nh % nkv != 0 || (bias != nullptr && n_dist <= 0) ||
        (gate != nullptr && gate_cols != 1 && gate_cols != dv))
        return RLIS_ERR_UNSUPPORTED;
    const long long n_rows = (long long)n_tokens * nh;
    if (n_rows > 0x7fffffffLL) return RLIS_ERR_UNSUPPORTED;
    const unsigned blocks = (unsigned)((n_rows + WARPS - 1) / WARPS);
    const size_t smem = (size_t)WARPS * d * sizeof(float);
    if (dtype == RLIS_F32)
        rlis_launch(attn_bias_kernel<float>, blocks, WARPS * 32, smem, stream, (const float*)q, (const float*)k_cache,
                    (const float*)v_cache, (float*)out, bias, n_dist, (const float*)gate, gate_stride, seq_of_token,
                    positions, block_tables, token_rows, max_blocks, (int)n_rows, nh, nkv, d, dv, page_size, scale, window,
                    sinks, slopes, gate_cols);
    else if (dtype == RLIS_BF16)
        rlis_launch(attn_bias_kernel<bf16>, blocks, WARPS * 32, smem, stream, (const bf16*)q, (const bf16*)k_cache,
                    (const bf16*)v_cache, (bf16*)out, bias, n_dist, (const bf16*)gate, gate_stride, seq_of_token,
                    positions, block_tables, token_rows, max_blocks, (int)n_rows, nh, nkv, d, dv, page_size, scale, window,
                    sinks, slopes, gate_cols);
    else
        return RLIS_ERR_UNSUPPORTED;
    return RLIS_LAUNCH_CHECK();
}

// A feed-forward that routes every token to `top` of `n_experts` small gated feed-forwards.
//
//   route:   z = W_r h (float32), s = sigmoid(z); the `top` experts with the largest s + correction are
//            chosen (ties: the lower index); their weights are s * route_scale (no renormalisation).  An
//            extra row of W_r, where given, is the logit of a gate on a shared expert: sigmoid of it.
//            With `softmax_chosen`: z = W_r h + b_r; the `top` experts with the largest z (+ correction) are
//            chosen and their weights are the softmax over the chosen logits alone, times route_scale.
//            scoring 2: s = softmax(z) over all router outputs.  `n_groups` > 1: the outputs form that many
//            equal groups of neighbours, a group's rank is its largest s + correction, and only outputs of the
//            `keep_groups` best groups can be chosen.  `normalize`: the chosen s are divided by their sum
//            (+ 1e-20) before route_scale.  Router outputs from `n_experts` of align and combine on (the last
//            rows of W_r) are identity experts: they have no matrices, and combine adds weight * x for them.
//   align:   the (token, choice) pairs are sorted by expert into slots; every expert's run of slots is
//            padded to a multiple of the row tile (32 rows, or 128 when there are many pairs an expert),
//            so a tile of rows belongs to one expert.  All on the device: no count ever reaches the
//            host, and launches depend on the step's shape only.
//   up:      act[slot, :] = glu(W_gate_e x, W_up_e x) for the slot's token x and expert e
//   down:    y[slot, :] = W_down_e act[slot, :]                         (float32)
//   combine: out[t, :] = sum_k weight[t, k] * y[slot(t, k), :] + shared_gate[t] * shared[t, :]
//
// glu(g, u) = g' * sigmoid(slope * g') * (u' + shift), g' = min(g, limit), u' = clamp(u, -limit, limit); slope +inf:
// max(g', 0) * (u' + shift).
//
// The products here are CUDA-core FFMA over k = 0..K-1 in that order for every output element, in float32
// whatever the element type, so a token's result does not depend on what else is in the batch; the
// tensor-core products for bfloat16 are in moe_mma.cu.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int BM = 32, BN = 64, BK = 16;     // the FFMA product's own tile; a row tile of the sort is a multiple of BM

__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }

// Four consecutive elements (from an address aligned to four of them) as floats, in one load.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}

// A CTA takes TOK tokens and has a warp for every row of W_r (up to 32 warps): a warp forms its row against
// all of the CTA's tokens, so the matrix is read once a CTA (the tokens' rows come back from the first-level
// cache) and the rows' sums run side by side; then one warp a token chooses.
template <typename T, int TOK>
__global__ __launch_bounds__(1024) void moe_route_kernel(
    const T* __restrict__ x, const float* __restrict__ w_router, const float* __restrict__ correction,
    int* __restrict__ top_idx, float* __restrict__ top_w, float* __restrict__ shared_gate,
    int n_tokens, int width, int n_experts, int top, float route_scale,
    const float* __restrict__ router_bias, int scoring, int n_groups, int keep_groups, int normalize) {
    pdl_wait_and_trigger();
    extern __shared__ float sm[];
    const bool softmax_chosen = scoring == 1;
    const int stride = 2 * n_experts + 1 + n_groups;   // per token: z [n_experts + 1], choice [n_experts], group ranks
    const int t0 = blockIdx.x * TOK;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int n_rows = n_experts + (shared_gate != nullptr ? 1 : 0);
    for (int e = warp; e < n_rows; e += nwarps) {
        const float* w = w_router + (size_t)e * width;
        float dot[TOK];
#pragma unroll
        for (int i = 0; i < TOK; ++i) dot[i] = 0.f;
        if ((width & 3) == 0) {
            // four elements a lane and step (16-byte loads of the matrix, four of a token's row)
#pragma unroll 4
            for (int k = lane * 4; k < width; k += 128) {
                const float4 wv = *reinterpret_cast<const float4*>(w + k);
#pragma unroll
                for (int i = 0; i < TOK; ++i) {
                    const int t = min(t0 + i, n_tokens - 1);
                    const float4 xv = load4(x + (size_t)t * width + k);
                    dot[i] = fmaf(wv.x, xv.x, dot[i]);
                    dot[i] = fmaf(wv.y, xv.y, dot[i]);
                    dot[i] = fmaf(wv.z, xv.z, dot[i]);
                    dot[i] = fmaf(wv.w, xv.w, dot[i]);
                }
            }
        } else {
#pragma unroll 4
            for (int k = lane; k < width; k += 32) {
                const float wv = w[k];
#pragma unroll
                for (int i = 0; i < TOK; ++i) {
                    const int t = min(t0 + i, n_tokens - 1);
                    dot[i] = fmaf(wv, to_f<T>(x[(size_t)t * width + k]), dot[i]);
                }
            }
        }
#pragma unroll
        for (int i = 0; i < TOK; ++i) {
            const float d = warp_sum(dot[i]);
            if (lane == 0) sm[i * stride + e] = d;
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < TOK * n_experts; idx += blockDim.x) {
        const int i = idx / n_experts, e = idx - i * n_experts;
        float* z = sm + i * stride;
        const float logit = z[e] + (router_bias != nullptr ? router_bias[e] : 0.f);
        const float s = scoring != 0 ? logit : sigmoidf_(logit);     // (scoring 2: the softmax is taken below)
        z[e] = s;
        z[n_experts + 1 + e] = s + (correction != nullptr ? correction[e] : 0.f);
    }
    if (threadIdx.x < TOK && shared_gate != nullptr && t0 + threadIdx.x < n_tokens)
        shared_gate[t0 + threadIdx.x] = sigmoidf_(sm[threadIdx.x * stride + n_experts]);
    __syncthreads();
    for (int i = warp; i < TOK; i += nwarps) {
        const int t = t0 + i;
        if (t >= n_tokens) break;
        float* z = sm + i * stride;
        float* choice = z + n_experts + 1;
        if (scoring == 2) {
            // softmax over all outputs, in float32; the correction joins the choice scores only
            float mx = -INFINITY;
            for (int e = lane; e < n_experts; e += 32) mx = fmaxf(mx, z[e]);
            mx = warp_max(mx);
            float sum = 0.f;
            for (int e = lane; e < n_experts; e += 32) sum += expf(z[e] - mx);
            sum = warp_sum(sum);
            for (int e = lane; e < n_experts; e += 32) {
                const float s = expf(z[e] - mx) / sum;
                z[e] = s;
                choice[e] = s + (correction != nullptr ? correction[e] : 0.f);
            }
            __syncwarp();
        }
        if (n_groups > 1) {
            // a group's rank is its best choice score; outputs of groups that are not kept cannot be chosen
            float* rank = choice + n_experts;
            const int per = n_experts / n_groups;
            for (int g = lane; g < n_groups; g += 32) {
                float r = -INFINITY;
                for (int e = g * per; e < (g + 1) * per; ++e) r = fmaxf(r, choice[e]);
                rank[g] = r;
            }
            __syncwarp();
            // a group is kept when fewer than keep_groups groups rank before it (ties: the lower index first)
            for (int g = lane; g < n_groups; g += 32) {
                const float r = rank[g];
                int before = 0;
                for (int o = 0; o < n_groups; ++o) before += (rank[o] > r || (rank[o] == r && o < g)) ? 1 : 0;
                if (before >= keep_groups)
                    for (int e = g * per; e < (g + 1) * per; ++e) choice[e] = -INFINITY;
            }
            __syncwarp();
        }
        for (int k = 0; k < top; ++k) {
            float best = -INFINITY;
            int at = 0x7fffffff;
            for (int e = lane; e < n_experts; e += 32) {
                const float c = choice[e];
                if (c > best || (c == best && e < at)) { best = c; at = e; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
            }
            if (at >= n_experts) at = k;        // scores that compare with nothing (NaN): still a valid index
            if (lane == 0) {
                top_idx[(size_t)t * top + k] = at;
                top_w[(size_t)t * top + k] = (softmax_chosen || normalize) ? z[at] : z[at] * route_scale;
                choice[at] = -INFINITY;
            }
            __syncwarp();
        }
        if (softmax_chosen && lane == 0) {
            // what is there so far are the chosen logits, the largest first
            float* wt = top_w + (size_t)t * top;
            const float zmax = wt[0];
            float sum = 0.f;
            for (int k = 0; k < top; ++k) {
                const float e = expf(wt[k] - zmax);
                wt[k] = e;
                sum += e;
            }
            for (int k = 0; k < top; ++k) wt[k] = wt[k] / sum * route_scale;
        } else if (normalize && lane == 0) {
            float* wt = top_w + (size_t)t * top;
            float sum = 0.f;
            for (int k = 0; k < top; ++k) sum += wt[k];
            for (int k = 0; k < top; ++k) wt[k] = wt[k] / (sum + 1e-20f) * route_scale;
        }
    }
}

// One CTA.  pairs = tokens * top.  sorted_pair [max_tiles * tile]: the pair in a slot or -1; pair_slot [pairs];
// tile_expert [max_tiles + 1]: the expert of a tile of `tile` slots or -1 (no such tile: they are the last
// ones), and after them the number of tiles that have one.
__global__ __launch_bounds__(1024) void moe_align_kernel(
    const int* __restrict__ top_idx, int* __restrict__ sorted_pair, int* __restrict__ pair_slot,
    int* __restrict__ tile_expert, int n_pairs, int n_experts, int max_tiles, int tile_rows) {
    pdl_wait_and_trigger();
    extern __shared__ int smi[];
    int* count = smi;                    // [n_experts]
    int* start = smi + n_experts;        // [n_experts]
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) count[e] = 0;
    for (int i = threadIdx.x; i < max_tiles * tile_rows; i += blockDim.x) sorted_pair[i] = -1;
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
        const int e = top_idx[i];
        if (e >= 0 && e < n_experts) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int tile = 0;
        for (int e = 0; e < n_experts; ++e) {
            start[e] = tile * tile_rows;
            const int tiles = (count[e] + tile_rows - 1) / tile_rows;
            for (int i = 0; i < tiles && tile < max_tiles; ++i) tile_expert[tile++] = e;
            count[e] = 0;                // from here on: the next free slot of the expert's run
        }
        tile_expert[max_tiles] = tile;
        for (; tile < max_tiles; ++tile) tile_expert[tile] = -1;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
        const int e = top_idx[i];
        if (e < 0 || e >= n_experts) { pair_slot[i] = -1; continue; }
        const int slot = start[e] + atomicAdd(&count[e], 1);
        if (slot >= max_tiles * tile_rows) { pair_slot[i] = -1; continue; }    // the host sizes max_tiles so that this never happens
        sorted_pair[slot] = i;
        pair_slot[i] = slot;
    }
}

// GLU true:  out[slot, n] = glu(A[token(slot), :] . Wg[e][n, :], A[token(slot), :] . Wu[e][n, :]), out in T
// GLU false: out[slot, n] = A[slot, :] . Wg[e][n, :], out float32
template <typename T, bool GLU>
__global__ __launch_bounds__(256) void moe_gemm_kernel(
    const T* __restrict__ A, const T* __restrict__ Wg, const T* __restrict__ Wu, void* __restrict__ out_,
    const int* __restrict__ sorted_pair, const int* __restrict__ tile_expert, int top, int N, int K,
    float slope, float limit, float shift, int tile_rows, long long w_stride, int il) {
    pdl_wait();
    const int e = tile_expert[blockIdx.y * BM / tile_rows];
    if (e < 0) return;
    __shared__ float As[BK][BM + 4];
    __shared__ float Gs[BK][BN + 4];
    __shared__ float Us[GLU ? BK : 1][BN + 4];
    __shared__ int rows[BM];
    const int slot0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    if (threadIdx.x < BM) {
        const int pair = sorted_pair[slot0 + threadIdx.x];
        rows[threadIdx.x] = pair < 0 ? -1 : (GLU ? pair / top : slot0 + (int)threadIdx.x);
    }
    __syncthreads();
    const T* wg = Wg + (size_t)e * w_stride;
    const T* wu = GLU ? Wu + (size_t)e * w_stride : nullptr;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float accg[2][4], accu[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) accg[i][j] = accu[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int i = threadIdx.x; i < BM * BK; i += 256) {
            const int r = i / BK, c = i % BK;
            const int gr = rows[r], gk = k0 + c;
            As[c][r] = (gr >= 0 && gk < K) ? to_f<T>(A[(size_t)gr * K + gk]) : 0.f;
        }
        for (int i = threadIdx.x; i < BN * BK; i += 256) {
            const int r = i / BK, c = i % BK;
            const int gn = n0 + r, gk = k0 + c;
            const bool in = gn < N && gk < K;
            // (il > 0: blocks of il gate rows, each followed by its il rows of the linear branch; Wu starts il rows in)
            const size_t wrow = il > 0 ? (size_t)(gn / il) * 2 * il + gn % il : (size_t)gn;
            Gs[c][r] = in ? to_f<T>(wg[wrow * K + gk]) : 0.f;
            if (GLU) Us[c][r] = in ? to_f<T>(wu[wrow * K + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[2], g[4], u[4];
#pragma unroll
            for (int i = 0; i < 2; ++i) a[i] = As[kk][ty * 2 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                g[j] = Gs[kk][tx * 4 + j];
                u[j] = GLU ? Us[kk][tx * 4 + j] : 0.f;
            }
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    accg[i][j] = fmaf(a[i], g[j], accg[i][j]);
                    if (GLU) accu[i][j] = fmaf(a[i], u[j], accu[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = ty * 2 + i;
        if (rows[r] < 0) continue;
        const size_t orow = (size_t)(slot0 + r) * N;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            if (GLU) {
                const float g = fminf(accg[i][j], limit);
                const float u = fminf(fmaxf(accu[i][j], -limit), limit);
                ((T*)out_)[orow + gn] = from_f<T>(glu_gate(g, slope) * (u + shift));
            } else {
                ((float*)out_)[orow + gn] = accg[i][j];
            }
        }
    }
    pdl_trigger();
}

template <typename T>
__global__ __launch_bounds__(256) void moe_combine_kernel(
    const float* __restrict__ y, const int* __restrict__ pair_slot, const float* __restrict__ top_w,
    const T* __restrict__ shared, const float* __restrict__ shared_gate, T* __restrict__ out, int width, int top,
    const T* __restrict__ x, const int* __restrict__ top_idx, int n_experts) {
    pdl_wait_and_trigger();
    const int t = blockIdx.x;
    const float sg = shared_gate != nullptr ? shared_gate[t] : 1.0f;
    if ((width & 3) == 0) {
        // four columns a thread: 16-byte loads of the slots' float32 rows; the same sums in the same order
        for (int c = threadIdx.x * 4; c < width; c += blockDim.x * 4) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int k = 0; k < top; ++k) {
                const int slot = pair_slot[(size_t)t * top + k];
                const bool same = slot < 0 && x != nullptr && top_idx[(size_t)t * top + k] >= n_experts;   // an identity expert
                if (slot < 0 && !same) continue;
                const float w = top_w[(size_t)t * top + k];
                const float4 v = same ? load4(x + (size_t)t * width + c)
                                      : *reinterpret_cast<const float4*>(y + (size_t)slot * width + c);
                acc.x = fmaf(w, v.x, acc.x); acc.y = fmaf(w, v.y, acc.y);
                acc.z = fmaf(w, v.z, acc.z); acc.w = fmaf(w, v.w, acc.w);
            }
            if (shared != nullptr) {
                const float4 v = load4(shared + (size_t)t * width + c);
                acc.x = fmaf(sg, v.x, acc.x); acc.y = fmaf(sg, v.y, acc.y);
                acc.z = fmaf(sg, v.z, acc.z); acc.w = fmaf(sg, v.w, acc.w);
            }
            T* o = out + (size_t)t * width + c;
            o[0] = from_f<T>(acc.x); o[1] = from_f<T>(acc.y); o[2] = from_f<T>(acc.z); o[3] = from_f<T>(acc.w);
        }
        return;
    }
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < top; ++k) {
            const int slot = pair_slot[(size_t)t * top + k];
            if (slot >= 0) acc = fmaf(top_w[(size_t)t * top + k], y[(size_t)slot * width + c], acc);
            else if (x != nullptr && top_idx[(size_t)t * top + k] >= n_experts)
                acc = fmaf(top_w[(size_t)t * top + k], to_f<T>(x[(size_t)t * width + c]), acc);
        }
        if (shared != nullptr) acc = fmaf(sg, to_f<T>(shared[(size_t)t * width + c]), acc);
        out[(size_t)t * width + c] = from_f<T>(acc);
    }
}

// interleave 0: gate in columns 0..I-1 and the linear branch in I..2I-1; interleave B > 0: blocks of B gate
// columns followed by their B columns of the linear branch (the layout the products' gated epilogues want).
template <typename T>
__global__ void glu_act_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter, size_t total,
                               float slope, float limit, float shift, int interleave) {
    pdl_wait_and_trigger();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t t = idx / inter;
    const int i = (int)(idx - t * inter);
    const size_t gi = interleave > 0 ? (size_t)(i / interleave) * 2 * interleave + i % interleave : (size_t)i;
    const size_t ui = interleave > 0 ? gi + interleave : (size_t)inter + i;
    const float g = fminf(to_f<T>(gu[t * 2 * inter + gi]), limit);
    const float u = fminf(fmaxf(to_f<T>(gu[t * 2 * inter + ui]), -limit), limit);
    out[idx] = from_f<T>(glu_gate(g, slope) * (u + shift));
}
}  // namespace


// x [T, width] in the element type; w_router float32 [n_experts (+ 1 with shared_gate), width];
// correction float32 [n_experts] or null; top_idx int32 [T, top]; top_w float32 [T, top]; shared_gate
// float32 [T] or null.  scoring 0: sigmoid; 1: softmax over the chosen logits; 2: softmax over all outputs.
extern "C" int rlis_moe_route(const void* x, const float* w_router, const float* correction, int* top_idx,
                              float* top_w, float* shared_gate, int n_tokens, int width, int n_experts, int top,
                              float route_scale, const float* router_bias, int scoring, int n_groups, int keep_groups,
                              int normalize, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (n_experts <= 0 || top <= 0 || top > n_experts || n_experts > 512 || scoring < 0 || scoring > 2) return RLIS_ERR_UNSUPPORTED;
    if (n_groups < 1 || n_experts % n_groups != 0 || keep_groups < 1 || keep_groups > n_groups ||
        top > keep_groups * (n_experts / n_groups) || (scoring == 2 && shared_gate != nullptr))
        return RLIS_ERR_UNSUPPORTED;
    // eight tokens a CTA when there are many (the router matrix is then read an eighth as often), one otherwise
    const int tok = n_tokens >= 64 ? 8 : 1;
    const size_t smem = (size_t)tok * (2 * n_experts + 1 + n_groups) * sizeof(float);
    if (smem > 48 * 1024) return RLIS_ERR_UNSUPPORTED;
    const unsigned blocks = (unsigned)((n_tokens + tok - 1) / tok);
    const int rows = n_experts + (shared_gate != nullptr ? 1 : 0);
    const unsigned threads = 32u * (unsigned)(rows < 32 ? (rows < tok ? tok : rows) : 32);
#define RLIS_ROUTE(T, TOK) rlis_launch(moe_route_kernel<T, TOK>, blocks, threads, smem, stream, (const T*)x, w_router, correction, \
                                       top_idx, top_w, shared_gate, n_tokens, width, n_experts, top, route_scale, \
                                       router_bias, scoring, n_groups, keep_groups, normalize)
    if (dtype == RLIS_F32) { if (tok == 8) RLIS_ROUTE(float, 8); else RLIS_ROUTE(float, 1); }
    else if (dtype == RLIS_BF16) { if (tok == 8) RLIS_ROUTE(bf16, 8); else RLIS_ROUTE(bf16, 1); }
    else return RLIS_ERR_UNSUPPORTED;
#undef RLIS_ROUTE
    return RLIS_LAUNCH_CHECK();
}

extern "C" int rlis_moe_align(const int* top_idx, int* sorted_pair, int* pair_slot, int* tile_expert, int n_pairs,
                              int n_experts, int max_tiles, int tile_rows, cudaStream_t stream) {
    if (n_pairs <= 0) return 0;
    if (n_experts <= 0 || n_experts > 4096 || tile_rows <= 0 || tile_rows % BM != 0 ||
        max_tiles < (n_pairs + tile_rows - 1) / tile_rows)
        return RLIS_ERR_UNSUPPORTED;
    rlis_launch(moe_align_kernel, 1, 1024, (size_t)2 * n_experts * sizeof(int), stream, top_idx, sorted_pair, pair_slot,
                tile_expert, n_pairs, n_experts, max_tiles, tile_rows);
    return RLIS_LAUNCH_CHECK();
}

// Rows of a step's tokens into slot order: out[slot, :] = x[token of the slot's pair, :], zeros in empty slots.
template <typename T>
__global__ __launch_bounds__(128) void moe_gather_rows_kernel(const T* __restrict__ x, T* __restrict__ out,
                                                              const int* __restrict__ sorted_pair, int top, int width) {
    pdl_wait_and_trigger();
    const int pair = sorted_pair[blockIdx.x];
    const T* src = pair >= 0 ? x + (size_t)(pair / top) * width : nullptr;
    T* dst = out + (size_t)blockIdx.x * width;
    constexpr int V = 16 / sizeof(T);
    if (width % V == 0) {
        const uint4* s4 = reinterpret_cast<const uint4*>(src);
        uint4* d4 = reinterpret_cast<uint4*>(dst);
        for (int i = threadIdx.x; i < width / V; i += blockDim.x) d4[i] = src != nullptr ? s4[i] : make_uint4(0u, 0u, 0u, 0u);
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = src != nullptr ? src[i] : from_f<T>(0.f);
    }
}

// glu != 0: A [T, K] rows of tokens, Wg and Wu [n_experts, N, K] (experts w_stride elements apart), out
// [max_tiles * tile_rows, N] in the element type.  interleave B > 0: gate and linear branch share one stack
// [n_experts, 2 N, K] in blocks of B gate rows, each followed by its B rows of the linear branch; Wg points
// at its first row and Wu B rows further.
// glu == 0: A [max_tiles * tile, K] rows of slots, Wg [n_experts, N, K], out float32 [max_tiles * tile, N].
extern "C" int rlis_moe_gemm(const void* A, const void* Wg, const void* Wu, void* out, const int* sorted_pair,
                             const int* tile_expert, int max_tiles, int tile_rows, int top, int N, int K, int glu,
                             float slope, float limit, float shift, long long w_stride, int interleave, int dtype,
                             cudaStream_t stream) {
    if (max_tiles <= 0 || N <= 0) return 0;
    if (tile_rows <= 0 || tile_rows % BM != 0 || interleave < 0 || (interleave > 0 && N % interleave != 0))
        return RLIS_ERR_UNSUPPORTED;
    dim3 grid((N + BN - 1) / BN, max_tiles * (tile_rows / BM));
    if (grid.y > 65535) return RLIS_ERR_UNSUPPORTED;
#define RLIS_MOE(T, G) rlis_launch(moe_gemm_kernel<T, G>, grid, 256, 0, stream, (const T*)A, (const T*)Wg, (const T*)Wu, \
                                   out, sorted_pair, tile_expert, top, N, K, slope, limit, shift, tile_rows, w_stride, interleave)
    if (dtype == RLIS_F32) { if (glu) RLIS_MOE(float, true); else RLIS_MOE(float, false); }
    else if (dtype == RLIS_BF16) { if (glu) RLIS_MOE(bf16, true); else RLIS_MOE(bf16, false); }
    else return RLIS_ERR_UNSUPPORTED;
#undef RLIS_MOE
    return RLIS_LAUNCH_CHECK();
}

// x [T, width] -> out [n_slots, width] in slot order (see moe_gather_rows_kernel).
extern "C" int rlis_moe_gather_rows(const void* x, void* out, const int* sorted_pair, int n_slots, int top, int width,
                                    int dtype, cudaStream_t stream) {
    if (n_slots <= 0 || width <= 0) return 0;
    if (dtype == RLIS_F32)
        rlis_launch(moe_gather_rows_kernel<float>, n_slots, 128, 0, stream, (const float*)x, (float*)out, sorted_pair, top, width);
    else if (dtype == RLIS_BF16)
        rlis_launch(moe_gather_rows_kernel<bf16>, n_slots, 128, 0, stream, (const bf16*)x, (bf16*)out, sorted_pair, top, width);
    else
        return RLIS_ERR_UNSUPPORTED;
    return RLIS_LAUNCH_CHECK();
}

extern "C" int rlis_moe_combine(const float* y, const int* pair_slot, const float* top_w, const void* shared,
                                const float* shared_gate, void* out, int n_tokens, int width, int top, const void* x,
                                const int* top_idx, int n_experts, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (dtype == RLIS_F32)
        rlis_launch(moe_combine_kernel<float>, n_tokens, 256, 0, stream, y, pair_slot, top_w, (const float*)shared,
                    shared_gate, (float*)out, width, top, (const float*)x, top_idx, n_experts);
    else if (dtype == RLIS_BF16)
        rlis_launch(moe_combine_kernel<bf16>, n_tokens, 256, 0, stream, y, pair_slot, top_w, (const bf16*)shared,
                    shared_gate, (bf16*)out, width, top, (const bf16*)x, top_idx, n_experts);
    else
        return RLIS_ERR_UNSUPPORTED;
    return RLIS_LAUNCH_CHECK();
}

// out[t, i] = glu(gate column i, linear column i of gu[t, :]); limit +inf: no clipping.
extern "C" int rlis_glu_act(const void* gu, void* out, int n_tokens, int inter, float slope, float limit, float shift,
                            int interleave, int dtype, cudaStream_t stream) {
    const size_t total = (size_t)n_tokens * inter;
    if (total == 0) return 0;
    if (interleave < 0 || (interleave > 0 && inter % interleave != 0)) return RLIS_ERR_UNSUPPORTED;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == RLIS_F32)
        rlis_launch(glu_act_kernel<float>, blocks, 256, 0, stream, (const float*)gu, (float*)out, inter, total, slope, limit, shift, interleave);
    else if (dtype == RLIS_BF16)
        rlis_launch(glu_act_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)gu, (bf16*)out, inter, total, slope, limit, shift, interleave);
    else
        return RLIS_ERR_UNSUPPORTED;
    return RLIS_LAUNCH_CHECK();
}

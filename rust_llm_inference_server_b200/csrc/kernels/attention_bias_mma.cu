// Tensor-core kernels (bfloat16) for the attention that attention_bias.cu describes: normed queries and
// keys, score = scale * q . k + bias[min(distance, n_dist - 1), head], keys of width D and values of
// width DV, a gate on every head's result; optionally slope_h * distance is subtracted from a score and
// exp(sink_h) joins the denominator of head h's softmax.  mma.sync m16n8k16 with float32 sums; keys and values reach
// shared memory by 16-byte asynchronous copies, two or three stages deep, in tiles of 64 keys; rows padded by 8
// elements so that ldmatrix is free of bank conflicts; softmax in float32 in units of log2(e).
//
// Portions of prompts: one CTA = one query head x 64 tokens of one request (4 warps x 16 rows); the
// causal edge is aligned to the end of the keys.  The bias of a tile depends on query - key only: the
// 127 distances of a 64 x 64 tile are brought to shared memory with the tile (times log2(e)); a tile
// that lies wholly beyond the table's reach adds the last row's constant instead.
//
// Single tokens: one CTA = one key/value head x one request x one piece of its context; the query
// heads of the group are the 16 rows of the products, so keys and values are read once a group.
// Each of the 4 warps takes 16 of a tile's 64 keys with a running softmax of its own; the warps are
// merged through shared memory at the end, pieces of a context by a second kernel.
#include "common.cuh"
#include "mma_utils.cuh"
#include <math.h>

namespace {
constexpr int WARPS = 4;
constexpr int THREADS = WARPS * 32;
constexpr int BM = 64;   // query tokens per CTA (prompts)
static_assert(BM == RLIS_PREFILL_TILE, "the host's tile list is cut for another tile size");
constexpr int BN = 64;   // keys per tile
constexpr float LOG2E = 1.4426950408889634f;

// 2^x in one instruction (relative error 2^-22; arguments here are at most 0, and -inf gives 0).
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int D, int DV> struct Stage { static constexpr int ELEMS = BN * (D + 8) + BN * (DV + 8); };
template <int D, int DV> constexpr size_t smem_bytes() {
    return (size_t)2 * Stage<D, DV>::ELEMS * sizeof(bf16) + 2 * 128 * sizeof(float);
}
// single tokens: three stages (two tiles of keys in flight while one is used: the kernel lives on bytes in flight)
constexpr int DEC_STAGES = 3;
template <int D, int DV> constexpr size_t decode_smem_bytes() {
    return (size_t)DEC_STAGES * Stage<D, DV>::ELEMS * sizeof(bf16);
}

// Brings tile `kt` of a request's keys and values into stage memory (ks_, vs_); keys outside [k_lo, k_hi) are zeros.
template <int D, int DV>
__device__ __forceinline__ void issue_tile(bf16* ks_, bf16* vs_, const bf16* kbase, const bf16* vbase,
                                           const int* table, int kt, int k_lo, int k_hi, int page_size,
                                           int page_shift, size_t page_stride_k, size_t page_stride_v) {
    // (page_shift: log2 of a power-of-two page size, or -1; a shift instead of a division a row)
    constexpr int CK = D / 8, CV = DV / 8;
#pragma unroll
    for (int i = 0; i < (BN * CK) / THREADS; ++i) {
        const int idx = threadIdx.x + i * THREADS;
        const int kin = idx / CK, c16 = idx % CK;
        const int key = kt * BN + kin;
        const bool valid = key < k_hi && key >= k_lo;
        size_t off = 0;
        if (valid) {
            const int pi = page_shift >= 0 ? key >> page_shift : key / page_size;
            off = (size_t)table[pi] * page_stride_k + (size_t)((key - pi * page_size) * D + c16 * 8);
        }
        cp_async16(ks_ + kin * (D + 8) + c16 * 8, kbase + off, valid);
    }
#pragma unroll
    for (int i = 0; i < (BN * CV) / THREADS; ++i) {
        const int idx = threadIdx.x + i * THREADS;
        const int kin = idx / CV, c16 = idx % CV;
        const int key = kt * BN + kin;
        const bool valid = key < k_hi && key >= k_lo;
        size_t off = 0;
        if (valid) {
            const int pi = page_shift >= 0 ? key >> page_shift : key / page_size;
            off = (size_t)table[pi] * page_stride_v + (size_t)((key - pi * page_size) * DV + c16 * 8);
        }
        cp_async16(vs_ + kin * (DV + 8) + c16 * 8, vbase + off, valid);
    }
}

// (four CTAs an SM for the narrow heads, three for the wide ones: the bound keeps the registers under that)
template <int D, int DV>
__global__ __launch_bounds__(THREADS, (D + DV <= 128) ? 4 : 3) void attn_bias_prefill_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
    bf16* __restrict__ out, const float* __restrict__ bias, int n_dist, const bf16* __restrict__ gate,
    long long gate_stride, const int* __restrict__ tiles, const int* __restrict__ cu_seqlens,
    const int* __restrict__ ctx_lens, const int* __restrict__ block_tables, int max_blocks, int nh, int nkv,
    int page_size, float scale, int window, const float* __restrict__ sinks, const float* __restrict__ slopes,
    int gate_cols) {
    pdl_wait();
    constexpr int SK = D + 8, SV = DV + 8;
    constexpr int KS = D / 16, ND = DV / 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* sbase = reinterpret_cast<bf16*>(smem_raw);
    float* bias_s = reinterpret_cast<float*>(sbase + 2 * Stage<D, DV>::ELEMS);     // [stage][128]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, c = lane & 3;
    const int b = tiles[2 * blockIdx.y], t0 = tiles[2 * blockIdx.y + 1];
    const int head = blockIdx.x;
    const int kvh = head / (nh / nkv);
    const int q_start = cu_seqlens[b];
    const int q_len = cu_seqlens[b + 1] - q_start;
    const int ctx = ctx_lens[b];
    const int start_pos = ctx - q_len;
    const int* table = block_tables + (size_t)b * max_blocks;

    const int r0 = warp * 16 + g, r1 = r0 + 8;            // this lane's two rows of the tile
    const int ti0 = t0 + r0, ti1 = t0 + r1;
    const bool rv0 = ti0 < q_len, rv1 = ti1 < q_len;
    const int pos0 = start_pos + ti0, pos1 = start_pos + ti1;
    const int lo0 = window > 0 ? max(0, pos0 - window + 1) : 0;
    const int lo1 = window > 0 ? max(0, pos1 - window + 1) : 0;

    uint32_t qa[KS][4];
    {
        const bf16* q0 = q + ((size_t)(q_start + (rv0 ? ti0 : 0)) * nh + head) * D;
        const bf16* q1 = q + ((size_t)(q_start + (rv1 ? ti1 : 0)) * nh + head) * D;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            qa[ks][0] = rv0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 2 * c) : 0u;
            qa[ks][1] = rv1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 2 * c) : 0u;
            qa[ks][2] = rv0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 2 * c + 8) : 0u;
            qa[ks][3] = rv1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 2 * c + 8) : 0u;
        }
    }
    const int last_tok = min(t0 + BM, q_len) - 1;
    const int k_hi = start_pos + last_tok + 1;                                  // exclusive
    const int k_lo = window > 0 ? max(0, start_pos + t0 - window + 1) : 0;
    const int kt0 = k_lo / BN, kt1 = (k_hi + BN - 1) / BN;
    const size_t psk = (size_t)nkv * page_size * D, psv = (size_t)nkv * page_size * DV;
    const int page_shift = (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1;
    const bf16* kbase = k_cache + (size_t)kvh * page_size * D;
    const bf16* vbase = v_cache + (size_t)kvh * page_size * DV;
    const float far_bias = bias != nullptr ? bias[(size_t)(n_dist - 1) * nh + head] * LOG2E : 0.f;
    const float slope_l2 = slopes != nullptr ? slopes[head] * LOG2E : 0.f;

    auto issue = [&](int kt, int stage) {
        bf16* ks_ = sbase + (size_t)stage * Stage<D, DV>::ELEMS;
        issue_tile<D, DV>(ks_, ks_ + BN * SK, kbase, vbase, table, kt, k_lo, k_hi, page_size, page_shift, psk, psv);
        // the tile's distances: row r, key column j are dist0 + r + (BN - 1 - j) apart
        const int dist0 = start_pos + t0 - (kt * BN + BN - 1);
        if (bias != nullptr && dist0 < n_dist - 1 && threadIdx.x < 2 * BN - 1) {
            const int dist = min(max(dist0 + (int)threadIdx.x, 0), n_dist - 1);
            bias_s[stage * 128 + threadIdx.x] = bias[(size_t)dist * nh + head] * LOG2E;
        }
        cp_async_commit();
    };

    const float scale_log2 = scale * LOG2E;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float oacc[ND][4];
#pragma unroll
    for (int nd = 0; nd < ND; ++nd)
#pragma unroll
        for (int e = 0; e < 4; ++e) oacc[nd][e] = 0.f;

    int stage = 0;
    if (kt0 < kt1) issue(kt0, 0);
    for (int kt = kt0; kt < kt1; ++kt) {
        if (kt + 1 < kt1) {
            issue(kt + 1, stage ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const bf16* ks_ = sbase + (size_t)stage * Stage<D, DV>::ELEMS;
        const bf16* vs_ = ks_ + BN * SK;
        const float* bs = bias_s + stage * 128;

        float sacc[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) sacc[nt][e] = 0.f;
#pragma unroll
            for (int ks2 = 0; ks2 < KS / 2; ++ks2) {
                uint32_t kb[4];
                ldmatrix_x4(kb, ks_ + (nt * 8 + (lane & 7)) * SK + ks2 * 32 + (lane >> 3) * 8);
                mma_bf16_16816(sacc[nt], qa[2 * ks2], kb[0], kb[1]);
                mma_bf16_16816(sacc[nt], qa[2 * ks2 + 1], kb[2], kb[3]);
            }
        }
        const bool edge = (kt + 1) * BN - 1 > start_pos + t0 + warp * 16 || window > 0;
        const bool near = bias != nullptr && start_pos + t0 - (kt * BN + BN - 1) < n_dist - 1;
        float mx0 = -INFINITY, mx1 = -INFINITY;
        if (!edge && !near && slopes == nullptr) {
            // most tiles of a long prompt: every key is seen by every row, and all share the table's last row
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float s0 = fmaf(sacc[nt][e], scale_log2, far_bias);
                    const float s1 = fmaf(sacc[nt][2 + e], scale_log2, far_bias);
                    sacc[nt][e] = s0;
                    sacc[nt][2 + e] = s1;
                    mx0 = fmaxf(mx0, s0);
                    mx1 = fmaxf(mx1, s1);
                }
        } else {
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int j = nt * 8 + 2 * c + e;
                    float s0 = fmaf(sacc[nt][e], scale_log2, near ? bs[r0 + BN - 1 - j] : far_bias);
                    float s1 = fmaf(sacc[nt][2 + e], scale_log2, near ? bs[r1 + BN - 1 - j] : far_bias);
                    const int key = kt * BN + j;
                    s0 = fmaf(slope_l2, (float)(key - pos0), s0);       // minus slope * distance
                    s1 = fmaf(slope_l2, (float)(key - pos1), s1);
                    if (edge) {
                        if (!(key <= pos0 && key >= lo0)) s0 = -INFINITY;
                        if (!(key <= pos1 && key >= lo1)) s1 = -INFINITY;
                    }
                    sacc[nt][e] = s0;
                    sacc[nt][2 + e] = s1;
                    mx0 = fmaxf(mx0, s0);
                    mx1 = fmaxf(mx1, s1);
                }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
        const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
        const float corr0 = ex2(m_run[0] - ms0), corr1 = ex2(m_run[1] - ms1);
        float ls0 = 0.f, ls1 = 0.f;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const float p0 = ex2(sacc[nt][e] - ms0), p1 = ex2(sacc[nt][2 + e] - ms1);
                sacc[nt][e] = p0;
                sacc[nt][2 + e] = p1;
                ls0 += p0;
                ls1 += p1;
            }
        ls0 += __shfl_xor_sync(0xffffffffu, ls0, 1);
        ls0 += __shfl_xor_sync(0xffffffffu, ls0, 2);
        ls1 += __shfl_xor_sync(0xffffffffu, ls1, 1);
        ls1 += __shfl_xor_sync(0xffffffffu, ls1, 2);
        l_run[0] = l_run[0] * corr0 + ls0;
        l_run[1] = l_run[1] * corr1 + ls1;
        m_run[0] = mn0;
        m_run[1] = mn1;
#pragma unroll
        for (int nd = 0; nd < ND; ++nd) {
            oacc[nd][0] *= corr0;
            oacc[nd][1] *= corr0;
            oacc[nd][2] *= corr1;
            oacc[nd][3] *= corr1;
        }
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
            uint32_t pa[4];
            pa[0] = pack_bf16(sacc[2 * kk][0], sacc[2 * kk][1]);
            pa[1] = pack_bf16(sacc[2 * kk][2], sacc[2 * kk][3]);
            pa[2] = pack_bf16(sacc[2 * kk + 1][0], sacc[2 * kk + 1][1]);
            pa[3] = pack_bf16(sacc[2 * kk + 1][2], sacc[2 * kk + 1][3]);
#pragma unroll
            for (int nd2 = 0; nd2 < ND / 2; ++nd2) {
                uint32_t vb[4];
                const int mat = lane >> 3;
                ldmatrix_x4_trans(vb, vs_ + (kk * 16 + (mat & 1) * 8 + (lane & 7)) * SV + (nd2 * 2 + (mat >> 1)) * 8);
                mma_bf16_16816(oacc[2 * nd2], pa, vb[0], vb[1]);
                mma_bf16_16816(oacc[2 * nd2 + 1], pa, vb[2], vb[3]);
            }
        }
        __syncthreads();       // everyone is done with this stage before the next copies land in it
        stage ^= 1;
    }

    if (sinks != nullptr) {
        // one more term of the denominator, without a key or a value (a sink far above every score gives inf, and 0)
        const float sink_l2 = sinks[head] * LOG2E;
        l_run[0] += ex2(sink_l2 - m_run[0]);
        l_run[1] += ex2(sink_l2 - m_run[1]);
    }
    float inv0 = l_run[0] > 0.f ? 1.0f / l_run[0] : 0.f;
    float inv1 = l_run[1] > 0.f ? 1.0f / l_run[1] : 0.f;
    const bool by_channel = gate != nullptr && gate_cols > 1;      // a logit a channel: gate[t, head * DV + col]
    if (gate != nullptr && !by_channel) {
        if (rv0) inv0 *= 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)(q_start + ti0) * gate_stride + head])));
        if (rv1) inv1 *= 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)(q_start + ti1) * gate_stride + head])));
    }
    if (rv0) {
        bf16* o = out + ((size_t)(q_start + ti0) * nh + head) * DV;
        const bf16* gr = by_channel ? gate + (size_t)(q_start + ti0) * gate_stride + (size_t)head * DV : nullptr;
#pragma unroll
        for (int nd = 0; nd < ND; ++nd) {
            float g0 = 1.0f, g1 = 1.0f;
            if (by_channel) {
                g0 = 1.0f / (1.0f + expf(-__bfloat162float(gr[nd * 8 + 2 * c])));
                g1 = 1.0f / (1.0f + expf(-__bfloat162float(gr[nd * 8 + 2 * c + 1])));
            }
            *reinterpret_cast<uint32_t*>(o + nd * 8 + 2 * c) = pack_bf16(oacc[nd][0] * inv0 * g0, oacc[nd][1] * inv0 * g1);
        }
    }
    if (rv1) {
        bf16* o = out + ((size_t)(q_start + ti1) * nh + head) * DV;
        const bf16* gr = by_channel ? gate + (size_t)(q_start + ti1) * gate_stride + (size_t)head * DV : nullptr;
#pragma unroll
        for (int nd = 0; nd < ND; ++nd) {
            float g0 = 1.0f, g1 = 1.0f;
            if (by_channel) {
                g0 = 1.0f / (1.0f + expf(-__bfloat162float(gr[nd * 8 + 2 * c])));
                g1 = 1.0f / (1.0f + expf(-__bfloat162float(gr[nd * 8 + 2 * c + 1])));
            }
            *reinterpret_cast<uint32_t*>(o + nd * 8 + 2 * c) = pack_bf16(oacc[nd][2] * inv1 * g0, oacc[nd][3] * inv1 * g1);
        }
    }
    pdl_trigger();
}

// partial [n_dec][nh][pieces][DV + 2] float32: unnormalised sums, then the maximum (log2 units) and the denominator.
template <int D, int DV>
__global__ __launch_bounds__(THREADS) void attn_bias_decode_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
    bf16* __restrict__ out, float* __restrict__ partial, const float* __restrict__ bias, int n_dist,
    const bf16* __restrict__ gate, long long gate_stride, const int* __restrict__ dec_rows,
    const int* __restrict__ dec_seqs, const int* __restrict__ ctx_lens, const int* __restrict__ block_tables,
    int max_blocks, int nh, int nkv, int page_size, float scale, int window, int pieces,
    const float* __restrict__ sinks, const float* __restrict__ slopes, int gate_cols) {
    pdl_wait();
    constexpr int SK = D + 8, SV = DV + 8;
    constexpr int KS = D / 16, ND = DV / 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* sbase = reinterpret_cast<bf16*>(smem_raw);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, c = lane & 3;
    const int kvh = blockIdx.x, bi = blockIdx.y, piece = blockIdx.z;
    const int nrep = nh / nkv;
    const int row = dec_rows[bi], seq = dec_seqs[bi];
    const int ctx = ctx_lens[seq];
    const int pos = ctx - 1;
    const int* table = block_tables + (size_t)seq * max_blocks;
    const int h0 = kvh * nrep + g, h1 = h0 + 8;            // this lane's two rows: heads of the group
    const bool rv0 = g < nrep, rv1 = g + 8 < nrep;

    uint32_t qa[KS][4];
    {
        const bf16* q0 = q + ((size_t)row * nh + (rv0 ? h0 : kvh * nrep)) * D;
        const bf16* q1 = q + ((size_t)row * nh + (rv1 ? h1 : kvh * nrep)) * D;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            qa[ks][0] = rv0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 2 * c) : 0u;
            qa[ks][1] = rv1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 2 * c) : 0u;
            qa[ks][2] = rv0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 2 * c + 8) : 0u;
            qa[ks][3] = rv1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 2 * c + 8) : 0u;
        }
    }
    const int k_lo = window > 0 ? max(0, ctx - window) : 0;
    const int k_hi = ctx;
    const int t_first = k_lo / BN, t_all = (k_hi + BN - 1) / BN - t_first;
    const int per = (t_all + pieces - 1) / pieces;
    const int kt0 = t_first + piece * per, kt1 = min(kt0 + per, t_first + t_all);
    const size_t psk = (size_t)nkv * page_size * D, psv = (size_t)nkv * page_size * DV;
    const int page_shift = (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1;
    const bf16* kbase = k_cache + (size_t)kvh * page_size * D;
    const bf16* vbase = v_cache + (size_t)kvh * page_size * DV;
    const float* brow0 = bias != nullptr ? bias + (rv0 ? h0 : 0) : nullptr;
    const float* brow1 = bias != nullptr ? bias + (rv1 ? h1 : 0) : nullptr;
    const float far0 = bias != nullptr ? brow0[(size_t)(n_dist - 1) * nh] * LOG2E : 0.f;
    const float far1 = bias != nullptr ? brow1[(size_t)(n_dist - 1) * nh] * LOG2E : 0.f;
    const float slope0 = slopes != nullptr && rv0 ? slopes[h0] * LOG2E : 0.f;
    const float slope1 = slopes != nullptr && rv1 ? slopes[h1] * LOG2E : 0.f;

    auto issue = [&](int kt, int stage) {
        bf16* ks_ = sbase + (size_t)stage * Stage<D, DV>::ELEMS;
        issue_tile<D, DV>(ks_, ks_ + BN * SK, kbase, vbase, table, kt, k_lo, k_hi, page_size, page_shift, psk, psv);
        cp_async_commit();
    };

    const float scale_log2 = scale * LOG2E;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float oacc[ND][4];
#pragma unroll
    for (int nd = 0; nd < ND; ++nd)
#pragma unroll
        for (int e = 0; e < 4; ++e) oacc[nd][e] = 0.f;

#pragma unroll
    for (int s = 0; s < DEC_STAGES - 1; ++s) {
        if (kt0 + s < kt1) issue(kt0 + s, s);
        else cp_async_commit();                      // an empty group keeps the count of groups in step
    }
    for (int kt = kt0; kt < kt1; ++kt) {
        const int stage = (kt - kt0) % DEC_STAGES;
        cp_async_wait<DEC_STAGES - 2>();
        __syncthreads();                             // tile kt has landed, and everyone is done with the stage of tile kt - 1
        if (kt + DEC_STAGES - 1 < kt1) issue(kt + DEC_STAGES - 1, (kt - kt0 + DEC_STAGES - 1) % DEC_STAGES);
        else cp_async_commit();
        const bf16* ks_ = sbase + (size_t)stage * Stage<D, DV>::ELEMS;
        const bf16* vs_ = ks_ + BN * SK;
        const int key0 = kt * BN + warp * 16;              // this warp's 16 keys of the tile
        if (key0 < k_hi && key0 + 15 >= k_lo) {
            float sacc[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) sacc[nt][e] = 0.f;
#pragma unroll
                for (int ks2 = 0; ks2 < KS / 2; ++ks2) {
                    uint32_t kb[4];
                    ldmatrix_x4(kb, ks_ + (warp * 16 + nt * 8 + (lane & 7)) * SK + ks2 * 32 + (lane >> 3) * 8);
                    mma_bf16_16816(sacc[nt], qa[2 * ks2], kb[0], kb[1]);
                    mma_bf16_16816(sacc[nt], qa[2 * ks2 + 1], kb[2], kb[3]);
                }
            }
            const bool near = bias != nullptr && pos - (key0 + 15) < n_dist - 1;
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int key = key0 + nt * 8 + 2 * c + e;
                    const bool seen = key < k_hi && key >= k_lo;
                    float b0 = far0, b1 = far1;
                    if (near && seen) {
                        const size_t at = (size_t)min(pos - key, n_dist - 1) * nh;
                        b0 = brow0[at] * LOG2E;
                        b1 = brow1[at] * LOG2E;
                    }
                    const float dist = (float)(key - pos);                   // minus the distance
                    const float s0 = seen ? fmaf(slope0, dist, fmaf(sacc[nt][e], scale_log2, b0)) : -INFINITY;
                    const float s1 = seen ? fmaf(slope1, dist, fmaf(sacc[nt][2 + e], scale_log2, b1)) : -INFINITY;
                    sacc[nt][e] = s0;
                    sacc[nt][2 + e] = s1;
                    mx0 = fmaxf(mx0, s0);
                    mx1 = fmaxf(mx1, s1);
                }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
            const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
            const float corr0 = exp2f(m_run[0] - ms0), corr1 = exp2f(m_run[1] - ms1);
            float ls0 = 0.f, ls1 = 0.f;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float p0 = exp2f(sacc[nt][e] - ms0), p1 = exp2f(sacc[nt][2 + e] - ms1);
                    sacc[nt][e] = p0;
                    sacc[nt][2 + e] = p1;
                    ls0 += p0;
                    ls1 += p1;
                }
            ls0 += __shfl_xor_sync(0xffffffffu, ls0, 1);
            ls0 += __shfl_xor_sync(0xffffffffu, ls0, 2);
            ls1 += __shfl_xor_sync(0xffffffffu, ls1, 1);
            ls1 += __shfl_xor_sync(0xffffffffu, ls1, 2);
            l_run[0] = l_run[0] * corr0 + ls0;
            l_run[1] = l_run[1] * corr1 + ls1;
            m_run[0] = mn0;
            m_run[1] = mn1;
#pragma unroll
            for (int nd = 0; nd < ND; ++nd) {
                oacc[nd][0] *= corr0;
                oacc[nd][1] *= corr0;
                oacc[nd][2] *= corr1;
                oacc[nd][3] *= corr1;
            }
            uint32_t pa[4];
            pa[0] = pack_bf16(sacc[0][0], sacc[0][1]);
            pa[1] = pack_bf16(sacc[0][2], sacc[0][3]);
            pa[2] = pack_bf16(sacc[1][0], sacc[1][1]);
            pa[3] = pack_bf16(sacc[1][2], sacc[1][3]);
#pragma unroll
            for (int nd2 = 0; nd2 < ND / 2; ++nd2) {
                uint32_t vb[4];
                const int mat = lane >> 3;
                ldmatrix_x4_trans(vb, vs_ + (warp * 16 + (mat & 1) * 8 + (lane & 7)) * SV + (nd2 * 2 + (mat >> 1)) * 8);
                mma_bf16_16816(oacc[2 * nd2], pa, vb[0], vb[1]);
                mma_bf16_16816(oacc[2 * nd2 + 1], pa, vb[2], vb[3]);
            }
        }
    }
    cp_async_wait<0>();
    __syncthreads();
    pdl_trigger();
    // the four warps' states meet in shared memory (the stages are free now): [warp][row][DV + 2]
    float* mg = reinterpret_cast<float*>(smem_raw);
    constexpr int MW = DV + 2;
    {
        float* a0 = mg + ((size_t)warp * 16 + g) * MW;
        float* a1 = a0 + 8 * MW;
#pragma unroll
        for (int nd = 0; nd < ND; ++nd) {
            a0[nd * 8 + 2 * c] = oacc[nd][0];
            a0[nd * 8 + 2 * c + 1] = oacc[nd][1];
            a1[nd * 8 + 2 * c] = oacc[nd][2];
            a1[nd * 8 + 2 * c + 1] = oacc[nd][3];
        }
        if (c == 0) {
            a0[DV] = m_run[0]; a0[DV + 1] = l_run[0];
            a1[DV] = m_run[1]; a1[DV + 1] = l_run[1];
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nrep * DV; idx += THREADS) {
        const int r = idx / DV, col = idx - r * DV;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) m = fmaxf(m, mg[((size_t)w * 16 + r) * MW + DV]);
        float l = 0.f, o = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float* a = mg + ((size_t)w * 16 + r) * MW;
            const float f = a[DV] == -INFINITY ? 0.f : exp2f(a[DV] - m);
            l = fmaf(a[DV + 1], f, l);
            o = fmaf(a[col], f, o);
        }
        const int head = kvh * nrep + r;
        if (pieces == 1) {
            if (sinks != nullptr) l += exp2f(sinks[head] * LOG2E - m);
            float inv = l > 0.f ? 1.0f / l : 0.f;
            if (gate != nullptr)
                inv *= 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)row * gate_stride + (gate_cols > 1 ? head * DV + col : head)])));
            out[((size_t)row * nh + head) * DV + col] = __float2bfloat16_rn(o * inv);
        } else {
            float* p = partial + (((size_t)bi * nh + head) * pieces + piece) * MW;
            p[col] = o;
            if (col == 0) { p[DV] = m; p[DV + 1] = l; }
        }
    }
}

// Pieces of a context into one result: one warp a (token, head).
__global__ __launch_bounds__(128) void attn_bias_decode_merge_kernel(
    const float* __restrict__ partial, bf16* __restrict__ out, const bf16* __restrict__ gate, long long gate_stride,
    const int* __restrict__ dec_rows, int n_units, int nh, int dv, int pieces, const float* __restrict__ sinks,
    int gate_cols) {
    pdl_wait_and_trigger();
    const int unit = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (unit >= n_units) return;
    const int bi = unit / nh, head = unit - bi * nh;
    const int row = dec_rows[bi];
    const int mw = dv + 2;
    const float* p = partial + (size_t)unit * pieces * mw;
    float m = -INFINITY;
    for (int s = 0; s < pieces; ++s) m = fmaxf(m, p[(size_t)s * mw + dv]);
    float l = 0.f;
    for (int s = 0; s < pieces; ++s) {
        const float ms = p[(size_t)s * mw + dv];
        l = fmaf(p[(size_t)s * mw + dv + 1], ms == -INFINITY ? 0.f : exp2f(ms - m), l);
    }
    if (sinks != nullptr) l += exp2f(sinks[head] * LOG2E - m);
    float inv = l > 0.f ? 1.0f / l : 0.f;
    const bool by_channel = gate != nullptr && gate_cols > 1;
    if (gate != nullptr && !by_channel) inv *= 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)row * gate_stride + head])));
    for (int col = lane; col < dv; col += 32) {
        float o = 0.f;
        for (int s = 0; s < pieces; ++s) {
            const float ms = p[(size_t)s * mw + dv];
            o = fmaf(p[(size_t)s * mw + col], ms == -INFINITY ? 0.f : exp2f(ms - m), o);
        }
        float gc = 1.0f;
        if (by_channel) gc = 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)row * gate_stride + (size_t)head * dv + col])));
        out[((size_t)row * nh + head) * dv + col] = __float2bfloat16_rn(o * inv * gc);
    }
}

bool sizes_taken(int d, int dv) { return (d == 64 || d == 128) && (dv == 32 || dv == 64 || dv == 128); }

template <int D, int DV> void raise_smem_limits() {
    cudaFuncSetAttribute(attn_bias_prefill_kernel<D, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes<D, DV>());
    cudaFuncSetAttribute(attn_bias_decode_kernel<D, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)decode_smem_bytes<D, DV>());
}
void raise_all_once() {
    static bool done = false;
    if (done) return;
    raise_smem_limits<64, 32>(); raise_smem_limits<64, 64>(); raise_smem_limits<64, 128>();
    raise_smem_limits<128, 32>(); raise_smem_limits<128, 64>(); raise_smem_limits<128, 128>();
    done = true;
}
}  // namespace

// Whether the kernels of this file exist for keys of width d and values of width dv (bfloat16).
extern "C" int rlis_attention_bias_mma_takes(int d, int dv) { return sizes_taken(d, dv) ? 1 : 0; }

#define RLIS_AB_DISPATCH(CALL)                                                         \
    if (d == 64 && dv == 32) { CALL(64, 32); } else if (d == 64 && dv == 64) { CALL(64, 64); } \
    else if (d == 64) { CALL(64, 128); } else if (dv == 32) { CALL(128, 32); }             \
    else if (dv == 64) { CALL(128, 64); } else { CALL(128, 128); }

// tiles: int32 [n_tiles][2] = (batch entry, first token of the tile within the entry's portion).
extern "C" int rlis_attention_bias_prefill(const void* q, const void* k_cache, const void* v_cache, void* out,
                                           const float* bias, int n_dist, const void* gate, long long gate_stride,
                                           const int* tiles, int n_tiles, const int* cu_seqlens, const int* ctx_lens,
                                           const int* block_tables, int max_blocks, int nh, int nkv, int d, int dv,
                                           int page_size, float scale, int window, const float* sinks,
                                           const float* slopes, int gate_cols, cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (!sizes_taken(d, dv) || nkv <= 0 || nh % nkv != 0 || n_tiles > 65535 || (bias != nullptr && n_dist <= 0) ||
        (gate != nullptr && gate_cols != 1 && gate_cols != dv))
        return RLIS_ERR_UNSUPPORTED;
    raise_all_once();
    dim3 grid(nh, n_tiles);
#define RLIS_AB_PF(D_, DV_) rlis_launch(attn_bias_prefill_kernel<D_, DV_>, grid, THREADS, smem_bytes<D_, DV_>(), stream, \
        (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out, bias, n_dist, (const bf16*)gate,      \
        gate_stride, tiles, cu_seqlens, ctx_lens, block_tables, max_blocks, nh, nkv, page_size, scale, window,        \
        sinks, slopes, gate_cols)
    RLIS_AB_DISPATCH(RLIS_AB_PF)
#undef RLIS_AB_PF
    return RLIS_LAUNCH_CHECK();
}

// partial: float32, at least n_dec * nh * pieces * (dv + 2) elements when pieces > 1.  sinks, slopes: float32 [nh] or null.
extern "C" int rlis_attention_bias_decode(const void* q, const void* k_cache, const void* v_cache, void* out,
                                          float* partial, const float* bias, int n_dist, const void* gate,
                                          long long gate_stride, const int* dec_rows, const int* dec_seqs,
                                          const int* ctx_lens, const int* block_tables, int max_blocks, int n_dec,
                                          int nh, int nkv, int d, int dv, int page_size, float scale, int window,
                                          int pieces, const float* sinks, const float* slopes, int gate_cols,
                                          cudaStream_t stream) {
    if (n_dec <= 0) return 0;
    if (!sizes_taken(d, dv) || nkv <= 0 || nh % nkv != 0 || nh / nkv > 16 || pieces < 1 || pieces > 65535 ||
        n_dec > 65535 || (bias != nullptr && n_dist <= 0) || (pieces > 1 && partial == nullptr) ||
        (gate != nullptr && gate_cols != 1 && gate_cols != dv))
        return RLIS_ERR_UNSUPPORTED;
    raise_all_once();
    dim3 grid(nkv, n_dec, pieces);
#define RLIS_AB_DEC(D_, DV_) rlis_launch(attn_bias_decode_kernel<D_, DV_>, grid, THREADS, decode_smem_bytes<D_, DV_>(), stream, \
        (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out, partial, bias, n_dist,                 \
        (const bf16*)gate, gate_stride, dec_rows, dec_seqs, ctx_lens, block_tables, max_blocks, nh, nkv, page_size,   \
        scale, window, pieces, sinks, slopes, gate_cols)
    RLIS_AB_DISPATCH(RLIS_AB_DEC)
#undef RLIS_AB_DEC
    int err = RLIS_LAUNCH_CHECK();
    if (err != 0 || pieces == 1) return err;
    const int units = n_dec * nh;
    rlis_launch(attn_bias_decode_merge_kernel, (units + 3) / 4, 128, 0, stream, (const float*)partial, (bf16*)out,
                (const bf16*)gate, gate_stride, dec_rows, units, nh, dv, pieces, sinks, gate_cols);
    return RLIS_LAUNCH_CHECK();
}

// The routed feed-forward's two products on the tensor cores (bfloat16; moe.cu describes the layer and
// holds the float32 products).  A tile of TM slots (32, or 128 when there are many pairs an expert)
// belongs to one expert (the sort pads every expert's run); a CTA forms TM slots x 64 features of it
// with mma.sync m16n8k16 and float32 sums, a warp 16 slots x 32 features (32 x 32 in the wide tiles, where
// a fragment of the weights then serves two of the slots' fragments).  Operands arrive by 16-byte
// asynchronous copies in steps of 64 along k through three stages, so two steps of weights are in
// flight while one is multiplied: with a few tokens a step the products are a stream of expert weights
// and live on bytes in flight.  The first product gathers its rows by token and forms gate and linear
// branch side by side, so the gating happens on the accumulators and neither branch reaches memory;
// the second reads the slots' rows and leaves float32.
#include "common.cuh"
#include "mma_utils.cuh"
#include <math.h>

namespace {
constexpr int TN = 64, TK = 64, SA = TK + 8, STAGES = 3;

template <bool GLU, int TM> struct MoeSmem { static constexpr int STAGE = (TM + TN * (GLU ? 2 : 1)) * SA; };

template <bool GLU, int TM>
__global__ __launch_bounds__(TM == 128 ? 256 : TM * 4) void moe_mma_kernel(
    const bf16* __restrict__ A, const bf16* __restrict__ Wg, const bf16* __restrict__ Wu, void* __restrict__ out_,
    const int* __restrict__ sorted_pair, const int* __restrict__ tile_expert, int top, int N, int K,
    float slope, float limit, float shift, long long w_stride, int il) {
    constexpr int MT = TM == 128 ? 2 : 1;            // fragments of 16 slots a warp
    constexpr int THREADS = TM * 4 / MT;             // TM / (16 MT) x 2 warps
    constexpr int STAGE = MoeSmem<GLU, TM>::STAGE;
    pdl_wait();
    const int e = tile_expert[blockIdx.y];
    if (e < 0) return;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* sm = reinterpret_cast<bf16*>(smem_raw);     // [stage][A: TM x SA | G: TN x SA | U: TN x SA]
    __shared__ int rows[TM];
    const int slot0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    if (threadIdx.x < TM) {
        const int pair = sorted_pair[slot0 + threadIdx.x];
        rows[threadIdx.x] = pair < 0 ? -1 : (GLU ? pair / top : slot0 + (int)threadIdx.x);
    }
    __syncthreads();
    const bf16* wg = Wg + (size_t)e * w_stride;
    const bf16* wu = GLU ? Wu + (size_t)e * w_stride : nullptr;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wm = warp >> 1, wn = warp & 1;         // a warp: 16 MT slots x 32 features
    const int g = lane >> 2, c = lane & 3;

    auto issue = [&](int k0, int st) {
        bf16* as = sm + (size_t)st * STAGE;
        bf16* gs = as + TM * SA;
        bf16* us = gs + TN * SA;
#pragma unroll
        for (int i = 0; i < (TM * 8) / THREADS; ++i) {      // TM rows x 8 chunks of 8
            const int idx = threadIdx.x + i * THREADS;
            const int r = idx >> 3, ch = idx & 7;
            const int gr = rows[r], gk = k0 + ch * 8;
            const bool ok = gr >= 0 && gk < K;
            cp_async16(as + r * SA + ch * 8, A + (ok ? (size_t)gr * K + gk : 0), ok);
        }
        constexpr int WCH = TN * 8 * (GLU ? 2 : 1);
#pragma unroll
        for (int i = 0; i < (WCH + THREADS - 1) / THREADS; ++i) {
            const int idx = threadIdx.x + i * THREADS;
            if (WCH % THREADS != 0 && idx >= WCH) break;
            const int which = idx / (TN * 8), rem = idx % (TN * 8);
            const int r = rem >> 3, ch = rem & 7;
            const int gn = n0 + r, gk = k0 + ch * 8;
            const bool ok = gn < N && gk < K;
            // (il 4: blocks of 4 gate rows, each followed by its 4 rows of the linear branch; wu starts 4 rows in)
            const size_t wrow = il == 4 ? (size_t)(((gn >> 2) << 3) + (gn & 3)) : (size_t)gn;
            const size_t off = ok ? wrow * K + gk : 0;
            cp_async16((which ? us : gs) + r * SA + ch * 8, (which ? wu : wg) + off, ok);
        }
        cp_async_commit();
    };

    float accg[MT][4][4], accu[MT][4][4];
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) accg[m][i][j] = accu[m][i][j] = 0.f;

    const int nk = (K + TK - 1) / TK;
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < nk) issue(s * TK, s);
        else cp_async_commit();                      // an empty group keeps the count of groups in step
    }
    for (int kt = 0; kt < nk; ++kt) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();                             // step kt has landed, and everyone is done with step kt - 1's stage
        if (kt + STAGES - 1 < nk) issue((kt + STAGES - 1) * TK, (kt + STAGES - 1) % STAGES);
        else cp_async_commit();
        const bf16* as = sm + (size_t)(kt % STAGES) * STAGE;
        const bf16* gs = as + TM * SA;
        const bf16* us = gs + TN * SA;
        uint32_t a[MT][4][4];
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
                ldmatrix_x4(a[m][kk], as + ((wm * MT + m) * 16 + (lane & 15)) * SA + kk * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int k2 = 0; k2 < 2; ++k2) {
                uint32_t b[4];
                ldmatrix_x4(b, gs + (wn * 32 + nt * 8 + (lane & 7)) * SA + k2 * 32 + (lane >> 3) * 8);
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    mma_bf16_16816(accg[m][nt], a[m][2 * k2], b[0], b[1]);
                    mma_bf16_16816(accg[m][nt], a[m][2 * k2 + 1], b[2], b[3]);
                }
                if (GLU) {
                    ldmatrix_x4(b, us + (wn * 32 + nt * 8 + (lane & 7)) * SA + k2 * 32 + (lane >> 3) * 8);
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        mma_bf16_16816(accu[m][nt], a[m][2 * k2], b[0], b[1]);
                        mma_bf16_16816(accu[m][nt], a[m][2 * k2 + 1], b[2], b[3]);
                    }
                }
            }
    }
    cp_async_wait<0>();
    pdl_trigger();
#pragma unroll
    for (int mh = 0; mh < 2 * MT; ++mh) {
        const int m = mh >> 1, half = mh & 1;
        const int r = (wm * MT + m) * 16 + g + half * 8;
        if (rows[r] < 0) continue;
        const size_t orow = (size_t)(slot0 + r) * N;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int gn = n0 + wn * 32 + nt * 8 + 2 * c + j;
                if (gn >= N) continue;
                const float vg = accg[m][nt][half * 2 + j];
                if (GLU) {
                    const float gg = fminf(vg, limit);
                    const float uu = fminf(fmaxf(accu[m][nt][half * 2 + j], -limit), limit);
                    ((bf16*)out_)[orow + gn] = __float2bfloat16_rn(glu_gate(gg, slope) * (uu + shift));
                } else {
                    ((float*)out_)[orow + gn] = vg;
                }
            }
    }
}

template <bool GLU, int TM>
int launch(const void* A, const void* Wg, const void* Wu, void* out, const int* sorted_pair, const int* tile_expert,
           int max_tiles, int top, int N, int K, float slope, float limit, float shift, long long w_stride, int il,
           cudaStream_t stream) {
    constexpr size_t smem = (size_t)STAGES * MoeSmem<GLU, TM>::STAGE * sizeof(bf16);
    static bool raised = false;
    if (!raised) {
        cudaFuncSetAttribute(moe_mma_kernel<GLU, TM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        raised = true;
    }
    dim3 grid((N + TN - 1) / TN, max_tiles);
    rlis_launch(moe_mma_kernel<GLU, TM>, grid, TM == 128 ? 256 : TM * 4, smem, stream, (const bf16*)A, (const bf16*)Wg, (const bf16*)Wu, out,
                sorted_pair, tile_expert, top, N, K, slope, limit, shift, w_stride, il);
    return RLIS_LAUNCH_CHECK();
}
}  // namespace

// The arguments of rlis_moe_gemm (moe.cu), for bfloat16 operands whose k extent is a multiple of 8 and row
// tiles of 32 or 128 slots.
extern "C" int rlis_moe_gemm_mma(const void* A, const void* Wg, const void* Wu, void* out, const int* sorted_pair,
                                 const int* tile_expert, int max_tiles, int tile_rows, int top, int N, int K, int glu,
                                 float slope, float limit, float shift, long long w_stride, int interleave,
                                 cudaStream_t stream) {
    if (max_tiles <= 0 || N <= 0) return 0;
    if (K % 8 != 0 || K <= 0 || max_tiles > 65535 || (tile_rows != 32 && tile_rows != 128) ||
        (interleave != 0 && interleave != 4) || (interleave == 4 && N % 4 != 0))
        return RLIS_ERR_UNSUPPORTED;
#define RLIS_MM(G, T) launch<G, T>(A, Wg, Wu, out, sorted_pair, tile_expert, max_tiles, top, N, K, slope, limit, shift, w_stride, interleave, stream)
    if (tile_rows == 32) return glu ? RLIS_MM(true, 32) : RLIS_MM(false, 32);
    return glu ? RLIS_MM(true, 128) : RLIS_MM(false, 128);
#undef RLIS_MM
}

extern "C" int rlis_moe_mma_takes_tile(int tile_rows) { return tile_rows == 32 || tile_rows == 128; }

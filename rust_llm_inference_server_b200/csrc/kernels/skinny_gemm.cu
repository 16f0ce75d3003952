// Weight-streaming matrix product for a handful of rows (decode): y[M, N] = x[M, K] W[N, K]^T,
// bf16 operands, float32 accumulation, M <= 16.  Every weight is read from HBM exactly once for
// all rows.  Role of the reference's small-batch GEMV (crates/model/src/gemv.metal:24-94: "each
// weight block read once for up to 8 rows"), on tensor cores.
//
// A CTA owns TN tiles of 8 output features and its 8 warps split K; a warp issues m16n8k16
// products with the rows of x as the M side (rows >= M are zero) and 8 features as the N side.
// Within a step of 32 k, lane (g, c) loads 16 bytes (8 consecutive k) of weight row g and of x
// rows g and g + 8 at k offset 8c; the two products of the step take elements 0..3 and 4..7 of
// those vectors.  The k index inside a product is thereby permuted in the same way for both
// operands, which a dot product does not see, and every load is a full 16-byte vector straight
// from global memory: a warp keeps all weight vectors of its share (TN x 8 steps) in flight at
// once.  The warps' partial sums meet in
// shared memory and are added in warp order (deterministic).
//
// (Two other arrangements were measured on the LM-head shape, 128256 x 2048, 8 rows, and lost:
// a persistent CTA per SM fed by cp.async.bulk copies through an mbarrier ring, 158 us, and a
// persistent CTA with register double-buffering, 131 us.  This one leans on many resident CTAs to
// hide the latency of the dependent tensor instructions and takes 110 us; the library GEMM takes
// 85 us, so products with very many output features are left to it, see ops.linear.)
//
// Epilogues: plain (bf16 or float32 out), or SwiGLU on a gate|up matrix whose rows are interleaved
// in blocks of 4 (rows 8t..8t+3 gate, 8t+4..8t+7 up): out[m, 4t + j] = silu(gate_j) * up_j.
#include "common.cuh"
#include "mma_utils.cuh"
#include <math.h>

namespace {
constexpr int SG_WARPS = 8;
constexpr int SG_THREADS = SG_WARPS * 32;
constexpr int SG_STEPS = 8;          // steps of 32 k per pass of a warp over its K share

__device__ __forceinline__ uint4 ldg16(const bf16* p) { return *reinterpret_cast<const uint4*>(p); }

template <typename OutT, int EPI, int TN>
__global__ __launch_bounds__(SG_THREADS) void skinny_gemm_kernel(const bf16* __restrict__ x,
                                                                 const bf16* __restrict__ W,
                                                                 OutT* __restrict__ y, int M, int N,
                                                                 int K, int ldy) {
    __shared__ float red[SG_WARPS][TN][16][8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, c = lane & 3;
    const int n0 = blockIdx.x * 8 * TN;
    const bool r0 = g < M, r1 = g + 8 < M;
    const bf16* x0 = x + (size_t)(r0 ? g : 0) * K;
    const bf16* x1 = x + (size_t)(r1 ? g + 8 : 0) * K;
    const bf16* wrow[TN];
    bool nvalid[TN];
#pragma unroll
    for (int t = 0; t < TN; ++t) {
        const int n = n0 + t * 8 + g;
        nvalid[t] = n < N;
        wrow[t] = W + (size_t)(nvalid[t] ? n : 0) * K;
    }
    const int steps_total = (K + 31) >> 5;
    const int spw = (steps_total + SG_WARPS - 1) / SG_WARPS;
    const int s0 = warp * spw, s1 = min(s0 + spw, steps_total);
    // two accumulators per tile: the tensor instructions of a pass form two chains, not one
    float acc[TN][2][4];
#pragma unroll
    for (int t = 0; t < TN; ++t)
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[t][h][e] = 0.f;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

    pdl_wait();
    for (int s = s0; s < s1; s += SG_STEPS) {
        uint4 wv[TN][SG_STEPS];
#pragma unroll
        for (int t = 0; t < TN; ++t)
#pragma unroll
            for (int u = 0; u < SG_STEPS; ++u) {
                const int k = ((s + u) << 5) + c * 8;
                wv[t][u] = ((s + u) < s1 && k + 8 <= K && nvalid[t]) ? ldg16(wrow[t] + k) : zero;
            }
#pragma unroll
        for (int u = 0; u < SG_STEPS; ++u) {
            const int k = ((s + u) << 5) + c * 8;
            const bool ok = (s + u) < s1 && k + 8 <= K;
            const uint4 xa = (ok && r0) ? ldg16(x0 + k) : zero;
            const uint4 xb = (ok && r1) ? ldg16(x1 + k) : zero;
            const uint32_t a_lo[4] = {xa.x, xb.x, xa.y, xb.y};
            const uint32_t a_hi[4] = {xa.z, xb.z, xa.w, xb.w};
#pragma unroll
            for (int t = 0; t < TN; ++t) {
                mma_bf16_16816(acc[t][0], a_lo, wv[t][u].x, wv[t][u].y);
                mma_bf16_16816(acc[t][1], a_hi, wv[t][u].z, wv[t][u].w);
            }
        }
    }
#pragma unroll
    for (int t = 0; t < TN; ++t) {
        red[warp][t][g][2 * c] = acc[t][0][0] + acc[t][1][0];
        red[warp][t][g][2 * c + 1] = acc[t][0][1] + acc[t][1][1];
        red[warp][t][g + 8][2 * c] = acc[t][0][2] + acc[t][1][2];
        red[warp][t][g + 8][2 * c + 1] = acc[t][0][3] + acc[t][1][3];
    }
    __syncthreads();
    if (EPI == 0) {
        for (int i = threadIdx.x; i < TN * 128; i += SG_THREADS) {
            const int t = i >> 7, m = (i >> 3) & 15, f = i & 7;
            const int n = n0 + t * 8 + f;
            if (m < M && n < N) {
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < SG_WARPS; ++w) v += red[w][t][m][f];
                y[(size_t)m * ldy + n] = from_f<OutT>(v);
            }
        }
    } else {
        for (int i = threadIdx.x; i < TN * 64; i += SG_THREADS) {
            const int t = i >> 6, m = (i >> 2) & 15, j = i & 3;
            const int nb = n0 + t * 8;
            if (m < M && nb + 4 + j < N) {
                float gt = 0.f, up = 0.f;
#pragma unroll
                for (int w = 0; w < SG_WARPS; ++w) {
                    gt += red[w][t][m][j];
                    up += red[w][t][m][4 + j];
                }
                const float sl = gt / (1.0f + expf(-gt));
                y[(size_t)m * ldy + (nb >> 1) + j] = from_f<OutT>(sl * up);
            }
        }
    }
    pdl_trigger();   // the next kernel of the stream may start its launch
}

template <typename OutT, int EPI>
void launch_skinny(const void* x, const void* W, void* y, int M, int N, int K, int ldy, cudaStream_t stream) {
    // (two feature tiles a CTA, TN = 2, measured slower at every size of the 1B model)
    rlis_launch(skinny_gemm_kernel<OutT, EPI, 1>, (unsigned)((N + 7) / 8), SG_THREADS, 0, stream,
                    (const bf16*)x, (const bf16*)W, (OutT*)y, M, N, K, ldy);
}
}  // namespace

// out_dtype: RLIS_BF16 or RLIS_F32.  epilogue 0: y [M, N]; epilogue 1 (SwiGLU, rows of W
// interleaved gate/up in blocks of 4): y [M, N / 2].
extern "C" int rlis_skinny_gemm_bf16(const void* x, const void* W, void* y, int M, int N, int K,
                                     int out_dtype, int epilogue, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 16 || K <= 0 || (K & 7) != 0) return RLIS_ERR_UNSUPPORTED;
    if (epilogue == 1 && (N & 7) != 0) return RLIS_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(W) & 15) != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0)
        return RLIS_ERR_UNSUPPORTED;            // 16-byte loads want aligned rows
    if (epilogue == 0 && out_dtype == RLIS_BF16)
        launch_skinny<bf16, 0>(x, W, y, M, N, K, N, stream);
    else if (epilogue == 0 && out_dtype == RLIS_F32)
        launch_skinny<float, 0>(x, W, y, M, N, K, N, stream);
    else if (epilogue == 1 && out_dtype == RLIS_BF16)
        launch_skinny<bf16, 1>(x, W, y, M, N, K, N / 2, stream);
    else
        return RLIS_ERR_UNSUPPORTED;
    return RLIS_LAUNCH_CHECK();
}

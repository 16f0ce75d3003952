// Weight-streaming matrix product for a handful of rows (decode): y[M, N] = x[M, K] W[N, K]^T,
// bf16 operands, float32 accumulation, M <= 16.  Every weight is read from HBM exactly once for
// all rows.  Role of the reference's small-batch GEMV (crates/model/src/gemv.metal:24-94: "each
// weight block read once for up to 8 rows"), on tensor cores.
//
// A CTA owns 8 output features and its 8 warps split K; a warp issues m16n8k16 products with the
// rows of x as the M side (rows >= M are zero) and the 8 features as the N side.  Within a step of
// 32 k, lane (g, c) loads 16 bytes (8 consecutive k) of weight row g and of x rows g and g + 8 at
// k offset 8c; the two products of the step take elements 0..3 and 4..7 of those chunks.  The
// k index inside a product is thereby permuted in the same way for both operands, which a dot
// product does not see, and every load is a full 16-byte vector straight from global memory.
// The warps' partial sums meet in shared memory and are added in warp order (deterministic).
//
// Epilogues: plain (bf16 or float32 out), or SwiGLU on a gate|up matrix whose rows are interleaved
// in blocks of 4 (rows 8t..8t+3 gate, 8t+4..8t+7 up): out[m, 4t + j] = silu(gate_j) * up_j.
#include "common.cuh"
#include "mma_utils.cuh"
#include <math.h>

namespace {
constexpr int SG_WARPS = 8;
constexpr int SG_THREADS = SG_WARPS * 32;
constexpr int SG_UNROLL = 4;

__device__ __forceinline__ uint4 ldg16(const bf16* p) { return *reinterpret_cast<const uint4*>(p); }

template <typename OutT, int EPI>
__global__ __launch_bounds__(SG_THREADS) void skinny_gemm_kernel(const bf16* __restrict__ x,
                                                                 const bf16* __restrict__ W,
                                                                 OutT* __restrict__ y, int M, int N,
                                                                 int K, int ldy) {
    __shared__ float red[SG_WARPS][16][8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, c = lane & 3;
    const int n0 = blockIdx.x * 8;
    const int n = n0 + g;
    const bool nvalid = n < N;
    const bf16* wrow = W + (size_t)(nvalid ? n : 0) * K;
    const bool r0 = g < M, r1 = g + 8 < M;
    const bf16* x0 = x + (size_t)(r0 ? g : 0) * K;
    const bf16* x1 = x + (size_t)(r1 ? g + 8 : 0) * K;

    const int steps_total = (K + 31) >> 5;
    const int spw = (steps_total + SG_WARPS - 1) / SG_WARPS;
    const int s0 = warp * spw, s1 = min(s0 + spw, steps_total);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

    for (int s = s0; s < s1; s += SG_UNROLL) {
        uint4 wv[SG_UNROLL], xa[SG_UNROLL], xb[SG_UNROLL];
#pragma unroll
        for (int u = 0; u < SG_UNROLL; ++u) {
            const int k = ((s + u) << 5) + c * 8;
            const bool ok = (s + u) < s1 && k + 8 <= K;
            wv[u] = (ok && nvalid) ? ldg16(wrow + k) : zero;
            xa[u] = (ok && r0) ? ldg16(x0 + k) : zero;
            xb[u] = (ok && r1) ? ldg16(x1 + k) : zero;
        }
#pragma unroll
        for (int u = 0; u < SG_UNROLL; ++u) {
            const uint32_t a_lo[4] = {xa[u].x, xb[u].x, xa[u].y, xb[u].y};
            const uint32_t a_hi[4] = {xa[u].z, xb[u].z, xa[u].w, xb[u].w};
            mma_bf16_16816(acc, a_lo, wv[u].x, wv[u].y);
            mma_bf16_16816(acc, a_hi, wv[u].z, wv[u].w);
        }
    }
    red[warp][g][2 * c] = acc[0];
    red[warp][g][2 * c + 1] = acc[1];
    red[warp][g + 8][2 * c] = acc[2];
    red[warp][g + 8][2 * c + 1] = acc[3];
    __syncthreads();
    if (EPI == 0) {
        if (threadIdx.x < 128) {
            const int m = threadIdx.x >> 3, f = threadIdx.x & 7;
            if (m < M && n0 + f < N) {
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < SG_WARPS; ++w) v += red[w][m][f];
                y[(size_t)m * ldy + n0 + f] = from_f<OutT>(v);
            }
        }
    } else {
        if (threadIdx.x < 64) {
            const int m = threadIdx.x >> 2, j = threadIdx.x & 3;
            if (m < M && n0 + 4 + j < N) {
                float gt = 0.f, up = 0.f;
#pragma unroll
                for (int w = 0; w < SG_WARPS; ++w) {
                    gt += red[w][m][j];
                    up += red[w][m][4 + j];
                }
                const float sl = gt / (1.0f + expf(-gt));
                y[(size_t)m * ldy + (n0 >> 1) + j] = from_f<OutT>(sl * up);
            }
        }
    }
}
}  // namespace

// out_dtype: RLIS_BF16 or RLIS_F32.  epilogue 0: y [M, N]; epilogue 1 (SwiGLU, rows of W
// interleaved gate/up in blocks of 4): y [M, N / 2].
extern "C" int rlis_skinny_gemm_bf16(const void* x, const void* W, void* y, int M, int N, int K,
                                     int out_dtype, int epilogue, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 16 || K <= 0 || (K & 7) != 0) return RLIS_ERR_UNSUPPORTED;
    if (epilogue == 1 && (N & 7) != 0) return RLIS_ERR_UNSUPPORTED;
    const unsigned grid = (unsigned)((N + 7) / 8);
    if (epilogue == 0 && out_dtype == RLIS_BF16)
        skinny_gemm_kernel<bf16, 0><<<grid, SG_THREADS, 0, stream>>>((const bf16*)x, (const bf16*)W, (bf16*)y, M, N, K, N);
    else if (epilogue == 0 && out_dtype == RLIS_F32)
        skinny_gemm_kernel<float, 0><<<grid, SG_THREADS, 0, stream>>>((const bf16*)x, (const bf16*)W, (float*)y, M, N, K, N);
    else if (epilogue == 1 && out_dtype == RLIS_BF16)
        skinny_gemm_kernel<bf16, 1><<<grid, SG_THREADS, 0, stream>>>((const bf16*)x, (const bf16*)W, (bf16*)y, M, N, K, N / 2);
    else
        return RLIS_ERR_UNSUPPORTED;
    return RLIS_LAUNCH_CHECK();
}

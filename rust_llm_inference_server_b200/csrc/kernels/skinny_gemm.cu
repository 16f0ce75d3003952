// Weight-streaming matrix product for a handful of rows (decode): y[M, N] = x[M, K] W[N, K]^T,
// bf16 operands, float32 accumulation, M <= 16.  Every weight is read from HBM exactly once for
// all rows.  Role of the reference's small-batch GEMV (crates/model/src/gemv.metal:24-94: "each
// weight block read once for up to 8 rows"), on tensor cores.
//
// A CTA owns 8 output features and its 8 warps split K; a warp issues m16n8k16 products with the
// rows of x as the M side (rows >= M are zero) and the 8 features as the N side.  Within a step of
// 32 k, lane (g, c) takes 16 bytes (8 consecutive k) of weight row g and of x rows g and g + 8 at
// k offset 8c; the two products of the step take elements 0..3 and 4..7 of those vectors.  The k
// index inside a product is thereby permuted in the same way for both operands, which a dot
// product does not see, and every access is a full 16-byte vector.  The weight vectors travel by
// cp.async into slots of shared memory that belong to the lane (16 steps = 8 KB a warp in flight,
// 64 KB a CTA: registers could not hold that much), so that a whole 2048-wide weight matrix of the
// decode step is in flight at once; x is small and comes from L1.  The warps' partial sums meet
// in shared memory and are added in warp order (deterministic).
//
// (Other arrangements were measured on the LM-head shape, 128256 x 2048, 8 rows, and lost:
// a persistent CTA per SM fed by cp.async.bulk copies through an mbarrier ring with the warps
// splitting K, 158 us; the same ring with each warp owning whole tiles (no sums across warps),
// 160 us: six warps an SM cannot hide the latency of the dependent tensor instructions and of
// the x loads; a persistent CTA with register double-buffering, 131 us.  This one, with two to
// seven CTAs of eight warps an SM, takes 97 us.  The library GEMM takes 85 us there, so
// products with very many output features are left to it, see ops.linear.)
//
// Epilogues: plain (bf16 or float32 out), or SwiGLU on a gate|up matrix whose rows are interleaved
// in blocks of 4 (rows 8t..8t+3 gate, 8t+4..8t+7 up): out[m, 4t + j] = silu(gate_j) * up_j.
#include "common.cuh"
#include "mma_utils.cuh"
#include <math.h>

namespace {
constexpr int SG_WARPS = 8;
constexpr int SG_THREADS = SG_WARPS * 32;
constexpr int SG_GROUP = 4;                         // steps of 32 k per cp.async group
// SG_GROUPS = groups a warp keeps in flight: 4 (16 steps = 8 KB a warp, 64 KB a CTA, three CTAs
// an SM) for matrices with few output features, where a CTA is all the parallelism there is;
// 2 (32 KB a CTA, seven CTAs an SM) where there are thousands of CTAs anyway.
template <typename OutT, int EPI, int SG_GROUPS>
__global__ __launch_bounds__(SG_THREADS) void skinny_gemm_kernel(const bf16* __restrict__ x,
                                                                 const bf16* __restrict__ W,
                                                                 OutT* __restrict__ y, int M, int N,
                                                                 int K, int ldy) {
    constexpr int SG_DEPTH = SG_GROUP * SG_GROUPS;
    extern __shared__ __align__(16) unsigned char sg_smem[];
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
    // this lane's private slots: slot u at (warp, u, lane); it reads back exactly what it copied,
    // so the layout is free of bank conflicts by construction
    uint4* slots = reinterpret_cast<uint4*>(sg_smem) + (size_t)warp * SG_DEPTH * 32 + lane;

    const int steps_total = (K + 31) >> 5;
    const int spw = (steps_total + SG_WARPS - 1) / SG_WARPS;
    const int s0 = warp * spw, s1 = min(s0 + spw, steps_total);
    // two accumulators: the tensor instructions of a pass form two chains, not one
    float acc0[4] = {0.f, 0.f, 0.f, 0.f}, acc1[4] = {0.f, 0.f, 0.f, 0.f};
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

    for (int base = s0; base < s1; base += SG_DEPTH) {
        // weights: no kernel writes them, so the first batch of copies may run ahead of pdl_wait
#pragma unroll
        for (int u = 0; u < SG_DEPTH; ++u) {
            const int k = ((base + u) << 5) + c * 8;
            const bool ok = (base + u) < s1 && k + 8 <= K && nvalid;
            cp_async16(slots + u * 32, wrow + (ok ? k : 0), ok);
            if ((u % SG_GROUP) == SG_GROUP - 1) cp_async_commit();
        }
        if (base == s0) pdl_wait();      // x comes from the kernel before
#pragma unroll
        for (int gi = 0; gi < SG_GROUPS; ++gi) {
            if (gi == 0) cp_async_wait<SG_GROUPS - 1>();
            if (gi == 1) cp_async_wait<(SG_GROUPS > 2 ? SG_GROUPS - 2 : 0)>();
            if (gi == 2) cp_async_wait<(SG_GROUPS > 3 ? SG_GROUPS - 3 : 0)>();
            if (gi == 3) cp_async_wait<0>();
            if (base + gi * SG_GROUP >= s1) continue;
#pragma unroll
            for (int v = 0; v < SG_GROUP; ++v) {
                const int u = gi * SG_GROUP + v;
                const int k = ((base + u) << 5) + c * 8;
                const bool ok = (base + u) < s1 && k + 8 <= K;
                const uint4 wv = slots[u * 32];
                const uint4 xa = (ok && r0) ? *reinterpret_cast<const uint4*>(x0 + k) : zero;
                const uint4 xb = (ok && r1) ? *reinterpret_cast<const uint4*>(x1 + k) : zero;
                const uint32_t a_lo[4] = {xa.x, xb.x, xa.y, xb.y};
                const uint32_t a_hi[4] = {xa.z, xb.z, xa.w, xb.w};
                mma_bf16_16816(acc0, a_lo, wv.x, wv.y);
                mma_bf16_16816(acc1, a_hi, wv.z, wv.w);
            }
        }
    }
    if (s0 >= s1) pdl_wait();
    red[warp][g][2 * c] = acc0[0] + acc1[0];
    red[warp][g][2 * c + 1] = acc0[1] + acc1[1];
    red[warp][g + 8][2 * c] = acc0[2] + acc1[2];
    red[warp][g + 8][2 * c + 1] = acc0[3] + acc1[3];
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
    pdl_trigger();   // the next kernel of the stream may start its launch
}

template <typename OutT, int EPI>
void launch_skinny(const void* x, const void* W, void* y, int M, int N, int K, int ldy, cudaStream_t stream) {
    constexpr size_t smem4 = (size_t)SG_WARPS * SG_GROUP * 4 * 32 * 16, smem2 = smem4 / 2;
    static bool attr_done = false;
    if (!attr_done) {
        cudaFuncSetAttribute(skinny_gemm_kernel<OutT, EPI, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem4);
        attr_done = true;
    }
    const unsigned grid = (unsigned)((N + 7) / 8);
    if (N < 8192)
        rlis_launch(skinny_gemm_kernel<OutT, EPI, 4>, grid, SG_THREADS, smem4, stream,
                    (const bf16*)x, (const bf16*)W, (OutT*)y, M, N, K, ldy);
    else
        rlis_launch(skinny_gemm_kernel<OutT, EPI, 2>, grid, SG_THREADS, smem2, stream,
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

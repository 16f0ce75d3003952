// bf16 matrix product on the fifth-generation tensor cores, for the prefill step:
//   y[M, N] = x[M, K] W[N, K]^T   (both operands K-major, as the checkpoint stores W)
// with the feed-forward's gating fused into the epilogue.  Role in the reference: the `matmul`
// calls of its tensor library (crates/model/src/layers.rs:82,181-184); here it is a hand-written
// sm_100a kernel so that SwiGLU never makes a round trip through HBM.
//
// One persistent CTA per SM walks over 128 x 256 tiles.  Six warps, by role:
//   warp 0, one lane: TMA producer.  Per k-block of 64 it asks for the 128 x 64 tile of x and the
//           256 x 64 tile of W (cp.async.bulk.tensor, 128-byte swizzle) into a ring of 4 stages;
//           an mbarrier per stage counts the bytes.
//   warp 1, one lane: issues tcgen05.mma (M 128, N 256, K 16, kind::f16) from shared-memory
//           descriptors into a 128 x 256 float32 accumulator in tensor memory; tcgen05.commit
//           hands a stage back to the producer when the products that read it have finished, and
//           tells the epilogue when the accumulator is complete.  The warp also owns the TMEM
//           allocation: all 512 columns, two accumulators, so that a tile's epilogue overlaps the
//           next tile's products.
//   warps 2-5: epilogue.  Each reads its quarter of the accumulator's lanes with tcgen05.ld, 32
//           columns at a time, and stores bf16 (or float32) rows, or silu(gate) * up for a gate|up
//           matrix whose rows are interleaved in blocks of 4.
// Rows and columns past M, N and K are zero-filled by TMA and never stored.
//
// Every mbarrier wait is bounded by a fifth of a second of wall time.  A wait that runs out sets an error word
// (rlis_gemm_tcgen05_error), lets every role run to its end without further waiting, and the
// CTA still frees its tensor memory before it returns.
#include "tcgen05_utils.cuh"
#include "gemm_epilogue.cuh"
#include <math.h>

namespace {
using namespace tc;
constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2, B_STAGE_BYTES = BN * BK * 2;
constexpr int GT_THREADS = 192;
constexpr size_t GT_SMEM = (size_t)STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + 1024 /* alignment */ + 256;

struct Ctrl {
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
    int abort;
};

constexpr uint32_t IDESC = idesc_bf16(BM, BN);

// EPI 0: bf16 y [M, N].  EPI 1: SwiGLU, y [M, N / 2] bf16.  EPI 2: float32 y [M, N].
// Persistent: CTA b works on tiles b, b + gridDim.x, ...; tile t -> (n tile t / m_tiles, m tile
// t % m_tiles), so the CTAs that run together share a few column blocks of W and all of x in L2.
// The accumulator is double-buffered in tensor memory (2 x 256 columns): the epilogue of a tile
// overlaps the products of the next one.
template <int EPI>
__global__ __launch_bounds__(GT_THREADS) void gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x,
                                                                  const __grid_constant__ CUtensorMap map_w,
                                                                  void* __restrict__ y, int M, int N, int K,
                                                                  int m_tiles, int num_tiles) {
    pdl_wait();
    extern __shared__ unsigned char gt_smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(gt_smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* a_tiles = base;
    unsigned char* b_tiles = base + (size_t)STAGES * A_STAGE_BYTES;
    Ctrl* ctrl = reinterpret_cast<Ctrl*>(b_tiles + (size_t)STAGES * B_STAGE_BYTES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        ctrl->abort = 0;
        for (int s = 0; s < STAGES; ++s) {
            bar_init(&ctrl->full[s], 1);
            bar_init(&ctrl->empty[s], 1);
        }
        for (int i = 0; i < 2; ++i) {
            bar_init(&ctrl->acc_full[i], 1);
            bar_init(&ctrl->acc_empty[i], 4);      // the four epilogue warps
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {   // all of tensor memory: two accumulators of 128 lanes x 256 float32 columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctrl->tmem_base)), "r"(2 * BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = ctrl->tmem_base;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            for (int tile = blockIdx.x; tile < num_tiles && !ctrl->abort; tile += gridDim.x) {
                const int n0 = (tile / m_tiles) * BN, m0 = (tile % m_tiles) * BM;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES && !bar_wait(&ctrl->empty[s], ((it / STAGES) - 1) & 1, &ctrl->abort)) break;
                    bar_expect_tx(&ctrl->full[s], A_STAGE_BYTES + B_STAGE_BYTES);
                    tma_load_2d(a_tiles + (size_t)s * A_STAGE_BYTES, &map_x, kb * BK, m0, &ctrl->full[s]);
                    tma_load_2d(b_tiles + (size_t)s * B_STAGE_BYTES, &map_w, kb * BK, n0, &ctrl->full[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int it = 0, t = 0;
            for (int tile = blockIdx.x; tile < num_tiles && !ctrl->abort; tile += gridDim.x, ++t) {
                const int buf = t & 1;
                if (t >= 2 && !bar_wait(&ctrl->acc_empty[buf], ((t >> 1) - 1) & 1, &ctrl->abort)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_acc = tmem_base + (uint32_t)(buf * BN);
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!bar_wait(&ctrl->full[s], (it / STAGES) & 1, &ctrl->abort)) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t adesc = smem_desc_sw128(a_tiles + (size_t)s * A_STAGE_BYTES);
                    const uint64_t bdesc = smem_desc_sw128(b_tiles + (size_t)s * B_STAGE_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)      // 32 bytes further along K in the swizzled row
                        umma_bf16(tmem_acc, adesc + (uint64_t)(k * UMMA_K * 2 >> 4), bdesc + (uint64_t)(k * UMMA_K * 2 >> 4),
                                  IDESC, (kb | k) != 0 ? 1u : 0u);
                    umma_commit(&ctrl->empty[s]);              // the stage is free once these products are done
                }
                umma_commit(&ctrl->acc_full[buf]);
            }
        }
    } else {
        // epilogue: warp w may touch TMEM lanes 32 * (w % 4) .. + 31
        const int q = warp & 3;
        int t = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++t) {
            const int buf = t & 1;
            const int n0 = (tile / m_tiles) * BN, m0 = (tile % m_tiles) * BM;
            const bool ok = bar_wait(&ctrl->acc_full[buf], (t >> 1) & 1, &ctrl->abort);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int row = m0 + q * 32 + lane;
            const uint32_t tmem_acc = tmem_base + (uint32_t)(buf * BN) + ((uint32_t)(q * 32) << 16);
            for (int cb = 0; cb < BN / 32; ++cb) {
                uint32_t r[32];
                tmem_ld32(tmem_acc + (uint32_t)(cb * 32), r);
                const int col = n0 + cb * 32;
                if (!ok || row >= M || col >= N) continue;
                store_sums32<EPI>(r, y, row, col, N);
            }
            // this warp has read its lanes of the buffer: hand it back to the product warp
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) bar_arrive(&ctrl->acc_empty[buf]);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * BN) : "memory");
    }
    pdl_trigger();   // the next kernel of the stream may start its launch
}

}  // namespace

#include "gemm_tcgen05_pair.cuh"

// 0 if no bounded wait of the tcgen05 product ever ran out on the current device.
extern "C" int rlis_gemm_tcgen05_error(void) {
    return tc::read_error_word();
}
extern "C" int* rlis_gemm_tcgen05_error_addr(void) { return tc::error_word_addr(); }

// epilogue 0: bf16 y [M, N]; 1: SwiGLU (rows of W interleaved gate/up in blocks of 4), bf16 y [M, N / 2];
// 2: float32 y [M, N].  K and N must be multiples of 8; pointers 16-byte aligned.
extern "C" int rlis_gemm_tcgen05(const void* x, const void* W, void* y, int M, int N, int K, int epilogue,
                                 cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || (K & 7) != 0 || (N & 7) != 0 || epilogue < 0 || epilogue > 2) return RLIS_ERR_UNSUPPORTED;
    if (epilogue == 1 && (N & 15) != 0) return RLIS_ERR_UNSUPPORTED;   // rows of N / 2 bf16 must stay 16-byte aligned
    if (((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(y)) & 15) != 0)
        return RLIS_ERR_UNSUPPORTED;
    // more than one tile of rows: two SMs to a tile of 256 x 256
    if (g_pair != 0 && M > BM) return launch_gemm_pair(x, W, y, M, N, K, epilogue, stream);
    CUtensorMap map_x, map_w;
    if (!make_map(&map_x, x, M, K, BM) || !make_map(&map_w, W, N, K, BN)) return RLIS_ERR_UNSUPPORTED;
    static bool attr_done = false;
    if (!attr_done) {
        cudaFuncSetAttribute(gemm_tcgen05_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GT_SMEM);
        cudaFuncSetAttribute(gemm_tcgen05_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GT_SMEM);
        cudaFuncSetAttribute(gemm_tcgen05_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GT_SMEM);
        attr_done = true;
    }
    const int m_tiles = (M + BM - 1) / BM, num_tiles = m_tiles * ((N + BN - 1) / BN);
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const unsigned grid = (unsigned)(num_tiles < sms ? num_tiles : sms);
    if (epilogue == 0)
        rlis_launch(gemm_tcgen05_kernel<0>, grid, GT_THREADS, GT_SMEM, stream, map_x, map_w, y, M, N, K, m_tiles, num_tiles);
    else if (epilogue == 1)
        rlis_launch(gemm_tcgen05_kernel<1>, grid, GT_THREADS, GT_SMEM, stream, map_x, map_w, y, M, N, K, m_tiles, num_tiles);
    else
        rlis_launch(gemm_tcgen05_kernel<2>, grid, GT_THREADS, GT_SMEM, stream, map_x, map_w, y, M, N, K, m_tiles, num_tiles);
    return RLIS_LAUNCH_CHECK();
}

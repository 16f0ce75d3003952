// The bf16 product y[M, N] = x[M, K] W[N, K]^T of gemm_tcgen05.cu with two SMs to a tile:
// `tcgen05.mma.cta_group::2`.  A cluster of two CTAs works on a tile of 256 x 256; CTA r of the
// pair holds rows 128 r .. 128 r + 127 of x and of the result (its own tensor memory), and HALF of
// the W tile (rows 128 r .. of the 256): the instruction, issued by one thread of CTA 0, reads each
// CTA's A tile from that CTA's shared memory and the B tile half from each.  Per k-block of 64 a
// CTA takes in 32 KB instead of 48 for the same 512 cycles of tensor work, so the 192 KB of a ring
// hold six blocks instead of four (the one-CTA kernel is bound by how far ahead its copies can be
// asked for: with three stages it is 8-15 % slower than with four), and the tensor core reads a
// third less from shared memory.
//
// Roles, in both CTAs unless said: warp 0 asks for the tiles (bulk tensor copies, 128-byte swizzle;
// the bytes of both CTAs are counted by CTA 0's barrier of the stage, `cp.async.bulk.tensor` with
// `.cta_group::2` and the barrier's address in the cluster's window); warp 1 of CTA 0 issues the
// instructions, `tcgen05.commit` with a mask of both CTAs hands a stage back to both producers and
// tells both epilogues when an accumulator is complete; warps 2-5 are the epilogue of their CTA's
// 128 rows (gemm_epilogue.cuh), and tell CTA 0 when they have read an accumulator.  Tensor memory:
// both CTAs' warp 1 allocate all 512 columns together (two accumulators of 256), and free them
// after the two CTAs have met at the end.
//
// Every mbarrier wait is bounded (tcgen05_utils.cuh); a wait that runs out sets the error word, every
// role runs to its end without further waits, the CTAs meet and free their tensor memory.
// (Included by gemm_tcgen05.cu, whose entry point chooses between the two kernels and whose error
// word this one shares.)
#pragma once
#include "tcgen05_utils.cuh"
#include "gemm_epilogue.cuh"
#include <math.h>

namespace {
using namespace tc;
constexpr int PM = 128;                 // rows of a CTA: the pair's tile is 2 PM x PN
constexpr int PN = 256, PK = 64, P_STAGES = 6;
constexpr int A_BYTES = PM * PK * 2, B_BYTES = (PN / 2) * PK * 2;       // 16 KB each a CTA and stage
constexpr int GP_THREADS = 192;
constexpr size_t GP_SMEM = (size_t)P_STAGES * (A_BYTES + B_BYTES) + 1024 /* alignment */ + 256;

struct PairCtrl {
    uint64_t full[P_STAGES];        // CTA 0's: both CTAs' bytes of a stage have arrived
    uint64_t empty[P_STAGES];       // each CTA's: the products that read the stage are done
    uint64_t acc_full[2];           // each CTA's: an accumulator is complete
    uint64_t acc_empty[2];          // CTA 0's: the eight epilogue warps of the pair have read it
    uint32_t tmem_base;
    int abort;
};
static_assert(sizeof(PairCtrl) <= 256, "the control block");

constexpr uint32_t IDESC_PAIR = idesc_bf16(2 * PM, PN);

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The address of a shared-memory object of CTA `rank` of the cluster, in the cluster's window.
__device__ __forceinline__ uint32_t in_cta(const void* p, uint32_t rank) {
    uint32_t a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(smem_u32(p)), "r"(rank));
    return a;
}
// A tile into this CTA's shared memory; its bytes are counted by the barrier at `bar_cluster_addr`,
// which may be the other CTA's of the pair.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, uint32_t bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// An arrival at the barrier at this offset in both CTAs of the pair once the products issued so far are done.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    const unsigned short both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(both) : "memory");
}
__device__ __forceinline__ void bar_arrive_cluster(uint32_t bar_cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

// Persistent: pair p works on tiles p, p + pairs, ...; tile t -> (n tile t / m_tiles, m tile t % m_tiles).
template <int EPI>
__global__ __launch_bounds__(GP_THREADS) void gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_x,
                                                                       const __grid_constant__ CUtensorMap map_w,
                                                                       void* __restrict__ y, int M, int N, int K,
                                                                       int m_tiles, int num_tiles) {
    pdl_wait();
    extern __shared__ unsigned char gp_smem_raw[];
    // the same offset in both CTAs (their dynamic arrays start at the same address): the instruction
    // reads both CTAs' tiles through one descriptor
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(gp_smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* a_tiles = base;
    unsigned char* b_tiles = base + (size_t)P_STAGES * A_BYTES;
    PairCtrl* ctrl = reinterpret_cast<PairCtrl*>(b_tiles + (size_t)P_STAGES * B_BYTES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int k_blocks = (K + PK - 1) / PK;

    if (threadIdx.x == 0) {
        ctrl->abort = 0;
        for (int s = 0; s < P_STAGES; ++s) {
            bar_init(&ctrl->full[s], 1);
            bar_init(&ctrl->empty[s], 1);
        }
        for (int i = 0; i < 2; ++i) {
            bar_init(&ctrl->acc_full[i], 1);
            bar_init(&ctrl->acc_empty[i], 8);      // the four epilogue warps of each CTA
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {   // one warp of each CTA of the pair: all of tensor memory in both
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctrl->tmem_base)), "r"(2 * PN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncwarp();
    cluster_sync_all();         // both CTAs' barriers exist before either is used from the other side
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = ctrl->tmem_base;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            for (int tile = pair; tile < num_tiles && !ctrl->abort; tile += pairs) {
                const int n0 = (tile / m_tiles) * PN, m0 = (tile % m_tiles) * 2 * PM;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % P_STAGES;
                    if (it >= P_STAGES && !bar_wait(&ctrl->empty[s], ((it / P_STAGES) - 1) & 1, &ctrl->abort)) break;
                    const uint32_t full0 = in_cta(&ctrl->full[s], 0);
                    if (rank == 0) bar_expect_tx(&ctrl->full[s], 2 * (A_BYTES + B_BYTES));
                    tma_load_2d_pair(a_tiles + (size_t)s * A_BYTES, &map_x, kb * PK, m0 + (int)rank * PM, full0);
                    tma_load_2d_pair(b_tiles + (size_t)s * B_BYTES, &map_w, kb * PK, n0 + (int)rank * (PN / 2), full0);
                }
            }
        }
    } else if (warp == 1) {
        if (rank == 0) {
            // The whole warp walks the loop and waits; one lane issues.  (Measured: the warp never
            // waits for a stage after the first, and a k-block still takes it 628 cycles for 512 of
            // tensor work: the instructions queue behind the pipe, which is held up by shared memory,
            // 32 KB a block written by the copies and 32 KB read by the products at 128 bytes a
            // cycle.  The kernel with one CTA a tile moves 48 + 48 KB a block and runs at 68 %.
            // Looking at the next stage's barrier ahead of the instructions changed nothing.  Tiles
            // of 192 columns, 128 of them in two rounds for a QKV product of 2048 x 3072 where tiles
            // of 256 are 96 in two rounds: 30.7 against 31.3 us, the bytes a k-block moves through
            // shared memory shrink by 15 % only.)
            int it = 0, t = 0;
            bool fine = true;
            for (int tile = pair; tile < num_tiles && fine && !ctrl->abort; tile += pairs, ++t) {
                const int buf = t & 1;
                if (t >= 2 && !bar_wait(&ctrl->acc_empty[buf], ((t >> 1) - 1) & 1, &ctrl->abort)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_acc = tmem_base + (uint32_t)(buf * PN);
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % P_STAGES;
                    if (!bar_wait(&ctrl->full[s], (it / P_STAGES) & 1, &ctrl->abort)) { fine = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    if (lane == 0) {
                        const uint64_t adesc = smem_desc_sw128(a_tiles + (size_t)s * A_BYTES);
                        const uint64_t bdesc = smem_desc_sw128(b_tiles + (size_t)s * B_BYTES);
#pragma unroll
                        for (int k = 0; k < PK / UMMA_K; ++k)      // 32 bytes further along K in the swizzled row
                            umma_bf16_pair(tmem_acc, adesc + (uint64_t)(k * UMMA_K * 2 >> 4), bdesc + (uint64_t)(k * UMMA_K * 2 >> 4),
                                           IDESC_PAIR, (kb | k) != 0 ? 1u : 0u);
                        umma_commit_pair(&ctrl->empty[s]);         // the stage is free in both CTAs once these are done
                    }
                    __syncwarp();
                }
                if (!fine) break;
                if (lane == 0) umma_commit_pair(&ctrl->acc_full[buf]);
                __syncwarp();
            }
        }
    } else {
        // epilogue: warp w may touch TMEM lanes 32 * (w % 4) .. + 31
        const int q = warp & 3;
        int t = 0;
        for (int tile = pair; tile < num_tiles; tile += pairs, ++t) {
            const int buf = t & 1;
            const int n0 = (tile / m_tiles) * PN, m0 = (tile % m_tiles) * 2 * PM + (int)rank * PM;
            const bool ok = bar_wait(&ctrl->acc_full[buf], (t >> 1) & 1, &ctrl->abort);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int row = m0 + q * 32 + lane;
            const uint32_t tmem_acc = tmem_base + (uint32_t)(buf * PN) + ((uint32_t)(q * 32) << 16);
            for (int cb = 0; cb < PN / 32; ++cb) {
                uint32_t r[32];
                tmem_ld32(tmem_acc + (uint32_t)(cb * 32), r);
                const int col = n0 + cb * 32;
                if (!ok || row >= M || col >= N) continue;
                store_sums32<EPI>(r, y, row, col, N);
            }
            // this warp has read its lanes of the buffer: CTA 0's product warp may write it again
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) bar_arrive_cluster(in_cta(&ctrl->acc_empty[buf], 0));
        }
    }
    // nobody leaves, and no tensor memory is freed, while the other CTA may still use this one's
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncwarp();
    cluster_sync_all();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * PN) : "memory");
    }
    pdl_trigger();
}

int g_pair = -1;        // -1: where the tiles allow; 0: never (measurements)
}  // namespace

extern "C" void rlis_gemm_tcgen05_set_pair(int on) { g_pair = on; }

// The same contract as rlis_gemm_tcgen05.// (the caller has checked the sizes and the alignment)
static int launch_gemm_pair(const void* x, const void* W, void* y, int M, int N, int K, int epilogue, cudaStream_t stream) {
    CUtensorMap map_x, map_w;
    if (!make_map(&map_x, x, M, K, PM) || !make_map(&map_w, W, N, K, PN / 2)) return RLIS_ERR_UNSUPPORTED;
    static bool attr_done = false;
    if (!attr_done) {
        cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GP_SMEM);
        cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GP_SMEM);
        cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GP_SMEM);
        attr_done = true;
    }
    const int m_tiles = (M + 2 * PM - 1) / (2 * PM), num_tiles = m_tiles * ((N + PN - 1) / PN);
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int pairs = num_tiles < sms / 2 ? num_tiles : sms / 2;
    const unsigned grid = (unsigned)(2 * pairs);
    const dim3 cluster(2, 1, 1);
    if (epilogue == 0)
        rlis_launch_cluster(gemm_tcgen05_pair_kernel<0>, dim3(grid), dim3(GP_THREADS), GP_SMEM, stream, cluster, map_x, map_w, y, M, N, K, m_tiles, num_tiles);
    else if (epilogue == 1)
        rlis_launch_cluster(gemm_tcgen05_pair_kernel<1>, dim3(grid), dim3(GP_THREADS), GP_SMEM, stream, cluster, map_x, map_w, y, M, N, K, m_tiles, num_tiles);
    else
        rlis_launch_cluster(gemm_tcgen05_pair_kernel<2>, dim3(grid), dim3(GP_THREADS), GP_SMEM, stream, cluster, map_x, map_w, y, M, N, K, m_tiles, num_tiles);
    return RLIS_LAUNCH_CHECK();
}

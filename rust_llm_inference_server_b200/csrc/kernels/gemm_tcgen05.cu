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
#include "common.cuh"
#include "mma_utils.cuh"
#include <cuda.h>
#include <math.h>

namespace {
constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2, B_STAGE_BYTES = BN * BK * 2;
constexpr int GT_THREADS = 192;
constexpr unsigned long long WAIT_LIMIT_NS = 200000000ull;   // a fifth of a second
constexpr size_t GT_SMEM = (size_t)STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + 1024 /* alignment */ + 256;

__device__ int g_gemm_error = 0;

__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void bar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void bar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait for the phase of the given parity; false (and `abort` set) when the bound ran out.
__device__ __forceinline__ bool bar_wait(uint64_t* bar, uint32_t parity, volatile int* abort) {
    const uint32_t addr = smem_u32(bar);
    if (*abort) return false;
    const unsigned long long t0 = now_ns();
    for (uint32_t spin = 0;; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
        if ((spin & 63u) == 63u && (*abort || now_ns() - t0 > WAIT_LIMIT_NS)) break;
    }
    *abort = 1;
    atomicExch(&g_gemm_error, 1);
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes wide, 128-byte swizzle:
// start address / 16 in bits 0-13, leading byte offset (unused by this layout) 1 in 16-29, stride
// between 8-row groups (1024 bytes) / 16 in 32-45, descriptor version 1 in 46-47, layout type 2
// (128-byte swizzle) in 61-63.
__device__ __forceinline__ uint64_t smem_desc_sw128(const void* tile) {
    const uint64_t addr = (uint64_t)(smem_u32(tile) >> 4) & 0x3FFFull;
    return addr | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor, kind::f16: float32 accumulator (bits 4-5 = 1), A and B bf16 (bits 7-9 and
// 10-12 = 1), both K-major (bits 15, 16 = 0), N / 8 in bits 17-22, M / 16 in bits 24-28.
constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(IDESC), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

struct Ctrl {
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
    int abort;
};

__device__ __forceinline__ void bar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

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
                                  (kb | k) != 0 ? 1u : 0u);
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
                if (EPI == 0) {
                    bf16* o = reinterpret_cast<bf16*>(y) + (size_t)row * N + col;
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        if (col + v * 8 >= N) break;
                        uint4 pk;
                        pk.x = pack_bf16(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]));
                        pk.y = pack_bf16(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
                        pk.z = pack_bf16(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
                        pk.w = pack_bf16(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
                        *reinterpret_cast<uint4*>(o + v * 8) = pk;
                    }
                } else if (EPI == 1) {
                    bf16* o = reinterpret_cast<bf16*>(y) + (size_t)row * (N >> 1) + (col >> 1);
                    float res[16];
#pragma unroll
                    for (int tt = 0; tt < 4; ++tt)
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float gt = __uint_as_float(r[tt * 8 + j]), up = __uint_as_float(r[tt * 8 + 4 + j]);
                            res[tt * 4 + j] = gt / (1.0f + expf(-gt)) * up;
                        }
#pragma unroll
                    for (int v = 0; v < 2; ++v) {
                        if (col + v * 16 >= N) break;
                        uint4 pk;
                        pk.x = pack_bf16(res[v * 8 + 0], res[v * 8 + 1]);
                        pk.y = pack_bf16(res[v * 8 + 2], res[v * 8 + 3]);
                        pk.z = pack_bf16(res[v * 8 + 4], res[v * 8 + 5]);
                        pk.w = pack_bf16(res[v * 8 + 6], res[v * 8 + 7]);
                        *reinterpret_cast<uint4*>(o + v * 8) = pk;
                    }
                } else {
                    float* o = reinterpret_cast<float*>(y) + (size_t)row * N + col;
#pragma unroll
                    for (int v = 0; v < 8; ++v) {
                        if (col + v * 4 >= N) break;
                        *reinterpret_cast<float4*>(o + v * 4) = make_float4(
                            __uint_as_float(r[v * 4]), __uint_as_float(r[v * 4 + 1]), __uint_as_float(r[v * 4 + 2]),
                            __uint_as_float(r[v * 4 + 3]));
                    }
                }
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

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// A [rows, K] bf16 row-major matrix as a 2-D tensor map with boxes of 64 k x box_rows rows, 128-byte swizzle.
bool make_map(CUtensorMap* map, const void* ptr, int rows, int K, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
}  // namespace

// 0 if no bounded wait of the tcgen05 product ever ran out on the current device.
extern "C" int rlis_gemm_tcgen05_error(void) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemm_error, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

// epilogue 0: bf16 y [M, N]; 1: SwiGLU (rows of W interleaved gate/up in blocks of 4), bf16 y [M, N / 2];
// 2: float32 y [M, N].  K and N must be multiples of 8; pointers 16-byte aligned.
extern "C" int rlis_gemm_tcgen05(const void* x, const void* W, void* y, int M, int N, int K, int epilogue,
                                 cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || (K & 7) != 0 || (N & 7) != 0 || epilogue < 0 || epilogue > 2) return RLIS_ERR_UNSUPPORTED;
    if (epilogue == 1 && (N & 15) != 0) return RLIS_ERR_UNSUPPORTED;   // rows of N / 2 bf16 must stay 16-byte aligned
    if (((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(y)) & 15) != 0)
        return RLIS_ERR_UNSUPPORTED;
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

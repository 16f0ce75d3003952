// Shared helpers for the sm_100a kernels: element conversion, 16-byte loads, warp reductions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

// Element type codes used by every exported launcher.
#define RLIS_F32 0
#define RLIS_BF16 1

// Tokens of a prompt portion that one CTA of the flash attention kernels takes.  The host cuts the
// step's tile list to this size (rlis_attention_prefill_tile); both kernels assert that they agree.
#define RLIS_PREFILL_TILE 64

// Error codes returned by launchers in addition to cudaError_t values (which are positive).
#define RLIS_ERR_UNSUPPORTED (-1)

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

// Number of elements of T in one 16-byte vector.
template <typename T> struct Vec16 { static constexpr int N = 16 / sizeof(T); };

// Loads 16 bytes from a 16-byte aligned address and widens them to float.
template <typename T> __device__ __forceinline__ void load16(const T* p, float* out);
template <> __device__ __forceinline__ void load16<float>(const float* p, float* out) {
    float4 v = *reinterpret_cast<const float4*>(p);
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
}
template <> __device__ __forceinline__ void load16<bf16>(const bf16* p, float* out) {
    uint4 v = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 f = __bfloat1622float2(h[i]);
        out[2 * i] = f.x;
        out[2 * i + 1] = f.y;
    }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float s = lane < nwarps ? scratch[lane] : 0.f;
        s = warp_sum(s);
        if (lane == 0) scratch[32] = s;
    }
    __syncthreads();
    float r = scratch[32];
    __syncthreads();
    return r;
}

// Rotate-half of the pair (a, b) = (x[j], x[j + d/2]) by the angle with cosine c and sine s, in
// float32 with the operations spelled out, so that every kernel that rotates gets the same bits.
__device__ __forceinline__ float rope_first(float a, float b, float c, float s) {
    return __fmaf_rn(a, c, -__fmul_rn(b, s));
}
__device__ __forceinline__ float rope_second(float a, float b, float c, float s) {
    return __fmaf_rn(b, c, __fmul_rn(a, s));
}

#define RLIS_LAUNCH_CHECK() ((int)cudaGetLastError())

// ---- programmatic dependent launch --------------------------------------------------------
// Every kernel of this library calls pdl_wait() before it touches anything an earlier kernel of
// the stream may write (or may still read), and pdl_trigger() when the next kernel may be launched
// beside it.  Launched with the programmatic-serialization attribute, the next kernel's CTAs then
// run their prologue (the first weight tiles of a weight-streaming product) before they wait for
// this kernel to finish; without the attribute both calls do nothing.  Before pdl_wait() a kernel
// may read only memory that no kernel of the step writes (weights, tensor maps) and write nothing.
// A kernel triggers only after its own wait: triggering at the top lets kernels pile up several
// deep, each holding SM slots while it waits, and the decode step ran a fifth slower that way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// For the short kernels of the decode step, and for those whose successor has weights to request:
// once this kernel's own dependency is resolved the next kernel may be launched beside it.  It runs
// its prologue (for the weight-streaming product: requests its first stages of weights) and then
// waits for this kernel to finish.  Only after the wait, so that never more than one kernel is
// queued up behind the running one.
__device__ __forceinline__ void pdl_wait_and_trigger() {
    pdl_wait();
    pdl_trigger();
}

extern int g_rlis_pdl;   // 1 (default): launches carry the attribute; see rlis_set_pdl in pdl.cu

template <typename... KArgs, typename... Args>
static inline void rlis_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                               cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_rlis_pdl ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same for a grid of thread-block clusters of `cluster` CTAs.
template <typename... KArgs, typename... Args>
static inline void rlis_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                       cudaStream_t stream, dim3 cluster, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster.x;
    attr[0].val.clusterDim.y = cluster.y;
    attr[0].val.clusterDim.z = cluster.z;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_rlis_pdl ? 2 : 1;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

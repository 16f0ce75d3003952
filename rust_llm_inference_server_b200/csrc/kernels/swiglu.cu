// SwiGLU gating: out[t, i] = silu(gate_i) * up_i, silu(z) = z * sigmoid(z), in float32, rounded
// once.  `gu` is the output of the fused gate|up projection ([tokens, 2I]).  interleave 0: gate
// in columns 0..I-1 and up in I..2I-1; interleave B > 0: blocks of B gate columns followed by
// their B up columns (the layout the decode kernel's fused epilogue wants).
// Formula: crates/model/src/layers.rs:181-184.
#include "common.cuh"

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter,
                              size_t total, int interleave) {
    pdl_wait();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    size_t t = idx / inter;
    int i = (int)(idx - t * inter);
    const size_t gi = interleave > 0 ? (size_t)(i / interleave) * 2 * interleave + i % interleave : (size_t)i;
    const size_t ui = interleave > 0 ? gi + interleave : (size_t)inter + i;
    float g = to_f<T>(gu[t * 2 * inter + gi]);
    float u = to_f<T>(gu[t * 2 * inter + ui]);
    float s = g / (1.0f + expf(-g));
    out[idx] = from_f<T>(s * u);
    pdl_trigger();   // the next kernel of the stream may start its launch
}

// bfloat16, blocks of 4: 16 bytes in (4 gate, 4 up), 8 bytes out per step; two steps a thread.
__global__ void swiglu_bf16_il4_kernel(const uint4* __restrict__ gu, uint2* __restrict__ out, size_t n_vec) {
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_vec) return;
    const uint4 v = gu[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    const float2 g01 = __bfloat1622float2(h[0]), g23 = __bfloat1622float2(h[1]);
    const float2 u01 = __bfloat1622float2(h[2]), u23 = __bfloat1622float2(h[3]);
    const float r0 = g01.x / (1.0f + expf(-g01.x)) * u01.x;
    const float r1 = g01.y / (1.0f + expf(-g01.y)) * u01.y;
    const float r2 = g23.x / (1.0f + expf(-g23.x)) * u23.x;
    const float r3 = g23.y / (1.0f + expf(-g23.y)) * u23.y;
    __nv_bfloat162 o01 = __floats2bfloat162_rn(r0, r1), o23 = __floats2bfloat162_rn(r2, r3);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&o01);
    o.y = *reinterpret_cast<uint32_t*>(&o23);
    out[i] = o;
    pdl_trigger();   // the next kernel of the stream may start its launch
}

extern "C" int rlis_swiglu(const void* gu, void* out, int n_tokens, int inter, int interleave,
                           int dtype, cudaStream_t stream) {
    size_t total = (size_t)n_tokens * inter;
    if (total == 0) return 0;
    if (interleave < 0 || (interleave > 0 && inter % interleave != 0)) return RLIS_ERR_UNSUPPORTED;
    const int threads = 256;
    if (dtype == RLIS_BF16 && interleave == 4) {
        const size_t n_vec = total / 4;      // inter % 4 == 0 was checked above
        rlis_launch(swiglu_bf16_il4_kernel, (unsigned)((n_vec + threads - 1) / threads), threads, 0, stream, 
            (const uint4*)gu, (uint2*)out, n_vec);
        return RLIS_LAUNCH_CHECK();
    }
    unsigned blocks = (unsigned)((total + threads - 1) / threads);
    if (dtype == RLIS_F32)
        rlis_launch(swiglu_kernel<float>, blocks, threads, 0, stream, (const float*)gu, (float*)out, inter, total, interleave);
    else if (dtype == RLIS_BF16)
        rlis_launch(swiglu_kernel<bf16>, blocks, threads, 0, stream, (const bf16*)gu, (bf16*)out, inter, total, interleave);
    else
        return RLIS_ERR_UNSUPPORTED;
    return RLIS_LAUNCH_CHECK();
}

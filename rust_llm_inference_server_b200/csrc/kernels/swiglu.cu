// SwiGLU gating: out[t, i] = silu(gate_i) * up_i, silu(z) = z * sigmoid(z), in float32, rounded
// once.  `gu` is the output of the fused gate|up projection ([tokens, 2I]).  interleave 0: gate
// in columns 0..I-1 and up in I..2I-1; interleave B > 0: blocks of B gate columns followed by
// their B up columns (the layout the decode kernel's fused epilogue wants).
// Formula: crates/model/src/layers.rs:181-184.
#include "common.cuh"

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter,
                              size_t total, int interleave) {
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
}

extern "C" int rlis_swiglu(const void* gu, void* out, int n_tokens, int inter, int interleave,
                           int dtype, cudaStream_t stream) {
    size_t total = (size_t)n_tokens * inter;
    if (total == 0) return 0;
    if (interleave < 0 || (interleave > 0 && inter % interleave != 0)) return RLIS_ERR_UNSUPPORTED;
    const int threads = 256;
    unsigned blocks = (unsigned)((total + threads - 1) / threads);
    if (dtype == RLIS_F32)
        swiglu_kernel<float><<<blocks, threads, 0, stream>>>((const float*)gu, (float*)out, inter, total, interleave);
    else if (dtype == RLIS_BF16)
        swiglu_kernel<bf16><<<blocks, threads, 0, stream>>>((const bf16*)gu, (bf16*)out, inter, total, interleave);
    else
        return RLIS_ERR_UNSUPPORTED;
    return RLIS_LAUNCH_CHECK();
}

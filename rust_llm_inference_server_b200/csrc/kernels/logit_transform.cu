// What an LM head may do to its float32 logits after the product: a scale, and a smooth cap
// cap * tanh(x / cap).  The reference's Llama does neither (crates/model/src/llama.rs:279-285:
// the product, cast to f32); the LM-head part launches this only when its spec asks for one.
#include "common.cuh"

namespace {
__global__ void logit_transform_kernel(float* __restrict__ logits, int vocab, long long row_stride,
                                       float scale, float cap) {
    pdl_wait_and_trigger();
    float* row = logits + (size_t)blockIdx.y * row_stride;
    const float inv_cap = cap > 0.f ? 1.f / cap : 0.f;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < vocab; i += gridDim.x * blockDim.x) {
        float x = row[i] * scale;
        if (cap > 0.f) x = cap * tanhf(x * inv_cap);
        row[i] = x;
    }
}
}  // namespace

// cap <= 0: no cap.
extern "C" int rlis_logit_transform(float* logits, int rows, int vocab, long long row_stride, float scale,
                                    float cap, cudaStream_t stream) {
    if (rows <= 0 || vocab <= 0) return 0;
    if (rows > 65535) return RLIS_ERR_UNSUPPORTED;
    const int threads = 256;
    int bx = (vocab + threads * 4 - 1) / (threads * 4);
    if (bx > 256) bx = 256;
    rlis_launch(logit_transform_kernel, dim3(bx, rows), dim3(threads), 0, stream, logits, vocab, row_stride, scale, cap);
    return RLIS_LAUNCH_CHECK();
}

// Negative log-likelihood of a target token per row of float32 logits:
//   nll[r] = log(sum_v exp(logit[r, v] - max)) + max - logit[r, target[r]]
// (the log_softmax + gather of the reference's perplexity, crates/engine/src/perplexity.rs:56-59).
#include "common.cuh"
#include <math.h>

namespace {
constexpr int NLL_THREADS = 512;

__global__ __launch_bounds__(NLL_THREADS) void nll_rows_kernel(const float* __restrict__ logits,
                                                               const int* __restrict__ targets,
                                                               float* __restrict__ nll, int vocab,
                                                               long long row_stride) {
    pdl_wait();
    __shared__ float scratch[33];
    const float* row = logits + (size_t)blockIdx.x * row_stride;
    float mx = -INFINITY;
    for (int v = threadIdx.x; v < vocab; v += NLL_THREADS) mx = fmaxf(mx, row[v]);
    mx = warp_max(mx);
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = mx;
    __syncthreads();
    if (threadIdx.x < 32) {
        float m = threadIdx.x < NLL_THREADS / 32 ? scratch[threadIdx.x] : -INFINITY;
        m = warp_max(m);
        if (threadIdx.x == 0) scratch[32] = m;
    }
    __syncthreads();
    mx = scratch[32];
    __syncthreads();
    float s = 0.f;
    for (int v = threadIdx.x; v < vocab; v += NLL_THREADS) s += expf(row[v] - mx);
    s = block_sum(s, scratch);
    if (threadIdx.x == 0) {
        const int t = targets[blockIdx.x];
        nll[blockIdx.x] = (t >= 0 && t < vocab) ? logf(s) + mx - row[t] : NAN;
    }
    pdl_trigger();   // the next kernel of the stream may start its launch
}
}  // namespace

extern "C" int rlis_nll_rows(const float* logits, const int* targets, float* nll, int rows, int vocab,
                             long long row_stride, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return RLIS_ERR_UNSUPPORTED;
    rlis_launch(nll_rows_kernel, rows, NLL_THREADS, 0, stream, logits, targets, nll, vocab, row_stride);
    return RLIS_LAUNCH_CHECK();
}

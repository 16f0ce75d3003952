// Repetition penalty on rows of float32 logits, in place, before the sampling kernels: every
// DISTINCT token of a request's history (prompt and output so far) has its logit divided by the
// penalty if it is positive, multiplied otherwise (crates/engine/src/sampler.rs:225-235; the
// reference does this on the host, on logits it has copied there).  One CTA per row: a bitmap of
// the vocabulary in shared memory tells the first thread that meets a token from the others that
// meet it again, so a repeated token is penalised once.
#include "common.cuh"

namespace {
__global__ __launch_bounds__(256) void repetition_penalty_kernel(float* __restrict__ logits,
                                                                 const int* __restrict__ rows,
                                                                 const int* __restrict__ history,
                                                                 const int* __restrict__ offsets,
                                                                 const float* __restrict__ penalties, int vocab,
                                                                 long long row_stride) {
    pdl_wait();
    extern __shared__ uint32_t seen[];
    const int r = blockIdx.x;
    const int words = (vocab + 31) >> 5;
    for (int i = threadIdx.x; i < words; i += blockDim.x) seen[i] = 0u;
    __syncthreads();
    float* row = logits + (size_t)rows[r] * row_stride;
    const float pen = penalties[r];
    const int lo = offsets[r], hi = offsets[r + 1];
    for (int i = lo + (int)threadIdx.x; i < hi; i += blockDim.x) {
        const int tok = history[i];
        if (tok < 0 || tok >= vocab) continue;
        const uint32_t bit = 1u << (tok & 31);
        if ((atomicOr(&seen[tok >> 5], bit) & bit) == 0u) {      // the first to meet this token
            const float l = row[tok];
            row[tok] = l > 0.f ? l / pen : l * pen;
        }
    }
    pdl_trigger();
}
}  // namespace

// logits float32 [*, vocab] with `row_stride` floats between rows; rows int32 [n]: the rows to
// penalise; history int32: the n requests' tokens one after the other, offsets int32 [n + 1] into
// it; penalties float32 [n].  Vocabularies up to 1.8 million (the bitmap lives in shared memory).
extern "C" int rlis_repetition_penalty(float* logits, const int* rows, const int* history, const int* offsets,
                                       const float* penalties, int n, int vocab, long long row_stride,
                                       cudaStream_t stream) {
    if (n <= 0) return 0;
    const size_t smem = (size_t)((vocab + 31) / 32) * 4;
    if (vocab <= 0 || smem > 227 * 1024) return RLIS_ERR_UNSUPPORTED;
    static bool attr_done = false;
    if (!attr_done) {
        cudaFuncSetAttribute(repetition_penalty_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        attr_done = true;
    }
    rlis_launch(repetition_penalty_kernel, (unsigned)n, 256, smem, stream, logits, rows, history, offsets, penalties,
                vocab, row_stride);
    return RLIS_LAUNCH_CHECK();
}

// RMSNorm over the float32 residual stream, fused with the residual addition that precedes it.
//
//   resid[t, :] += delta[t, :]            (only when delta is given; float32 sum, stored as float32)
//   out[t, :]    = resid[t, :] / sqrt(mean(resid[t, :]^2) + eps) * w     (rounded once to T)
//
// With a row list, output row i is computed from source row rows[i] (the rows whose logits are
// wanted) and the residual stream is left as it is.
//
// Formula: crates/model/src/layers.rs:141-146 (weight multiplies directly, eps as float32);
// the residual additions are crates/model/src/llama.rs:267,270.  Sum of squares and scale in
// float32; the order of the sum depends only on the width, never on the batch.
#include "common.cuh"

template <typename T>
__global__ void rmsnorm_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                               const float* __restrict__ w, T* __restrict__ out,
                               const int* __restrict__ rows, int hidden, float eps) {
    __shared__ float scratch[33];
    const size_t obase = (size_t)blockIdx.x * hidden;
    if (rows != nullptr) {
        const size_t base = (size_t)rows[blockIdx.x] * hidden;
        float ss = 0.f;
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            float v = resid[base + i] + (delta != nullptr ? to_f<T>(delta[base + i]) : 0.f);
            ss += v * v;
        }
        ss = block_sum(ss, scratch);
        const float rstd = 1.0f / sqrtf(ss / (float)hidden + eps);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            float v = resid[base + i] + (delta != nullptr ? to_f<T>(delta[base + i]) : 0.f);
            out[obase + i] = from_f<T>(v * rstd * w[i]);
        }
        return;
    }
    const size_t base = obase;
    float ss = 0.f;
    if (delta != nullptr) {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            float v = resid[base + i] + to_f<T>(delta[base + i]);
            resid[base + i] = v;
            ss += v * v;
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            float v = resid[base + i];
            ss += v * v;
        }
    }
    ss = block_sum(ss, scratch);
    const float rstd = 1.0f / sqrtf(ss / (float)hidden + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        out[base + i] = from_f<T>(resid[base + i] * rstd * w[i]);
}

extern "C" int rlis_rmsnorm(float* resid, const void* delta, const float* w, void* out,
                            const int* rows, int n_tokens, int hidden, float eps, int dtype,
                            cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    if (dtype == RLIS_F32)
        rmsnorm_kernel<float><<<n_tokens, threads, 0, stream>>>(resid, (const float*)delta, w, (float*)out, rows, hidden, eps);
    else if (dtype == RLIS_BF16)
        rmsnorm_kernel<bf16><<<n_tokens, threads, 0, stream>>>(resid, (const bf16*)delta, w, (bf16*)out, rows, hidden, eps);
    else
        return RLIS_ERR_UNSUPPORTED;
    return RLIS_LAUNCH_CHECK();
}

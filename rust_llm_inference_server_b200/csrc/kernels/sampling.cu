// Token selection on the device: one token per row of float32 logits, greedy or by the Gumbel-max
// trick with counter-based noise, so only token ids leave the GPU.
//
// Same definition as the reference's CPU code (crates/model/src/sampling.rs:11-23,54-63,86-100):
//   h = lowbias32(key ^ v * 0x9e3779b9);  u = ((h >> 9) + 0.5) * 2^-23  (23 bits: never 1.0)
//   score(v) = logit[v] * (1/T) - log(-log u);  the highest score wins, ties go to the lowest id.
// params[r] = (key, bits of 1/T as float); (0, 0) means greedy.  A row's choice depends on its
// own logits and key only, never on its neighbours in the batch.
#include "common.cuh"
#include <math.h>

namespace {
__device__ __forceinline__ uint32_t lowbias32(uint32_t x) {
    x ^= x >> 16;
    x *= 0x7feb352du;
    x ^= x >> 15;
    x *= 0x846ca68bu;
    x ^= x >> 16;
    return x;
}

__device__ __forceinline__ bool better(float s, int v, float bs, int bv) {
    return s > bs || (s == bs && v < bv);
}

constexpr int THREADS = 512;

__global__ __launch_bounds__(THREADS) void sample_rows_kernel(const float* __restrict__ logits,
                                                              const uint32_t* __restrict__ params,
                                                              int* __restrict__ out, int vocab,
                                                              long long row_stride) {
    __shared__ float s_val[THREADS / 32];
    __shared__ int s_idx[THREADS / 32];
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * row_stride;
    const uint32_t key = params[2 * r];
    const float inv_t = __uint_as_float(params[2 * r + 1]);
    float best = -INFINITY;
    int best_v = 0x7fffffff;
    for (int v = threadIdx.x; v < vocab; v += THREADS) {
        float s = row[v];
        if (inv_t > 0.f) {
            const uint32_t h = lowbias32(key ^ ((uint32_t)v * 0x9e3779b9u));
            const float u = __fmul_rn((float)(h >> 9) + 0.5f, 1.0f / 8388608.0f);
            const float g = -logf(-logf(u));
            s = __fadd_rn(__fmul_rn(s, inv_t), g);
        }
        if (better(s, v, best, best_v)) { best = s; best_v = v; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float os = __shfl_xor_sync(0xffffffffu, best, o);
        const int ov = __shfl_xor_sync(0xffffffffu, best_v, o);
        if (better(os, ov, best, best_v)) { best = os; best_v = ov; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { s_val[warp] = best; s_idx[warp] = best_v; }
    __syncthreads();
    if (warp == 0) {
        best = lane < THREADS / 32 ? s_val[lane] : -INFINITY;
        best_v = lane < THREADS / 32 ? s_idx[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float os = __shfl_xor_sync(0xffffffffu, best, o);
            const int ov = __shfl_xor_sync(0xffffffffu, best_v, o);
            if (better(os, ov, best, best_v)) { best = os; best_v = ov; }
        }
        // A row of NaNs or -inf leaves best_v at its sentinel: report id 0 as the reference's
        // argmax does (crates/engine/src/sampler.rs:238-246 starts from index 0).
        if (lane == 0) out[r] = best_v == 0x7fffffff ? 0 : best_v;
    }
}
}  // namespace

extern "C" int rlis_sample_rows(const float* logits, const uint32_t* params, int* out, int rows,
                                int vocab, long long row_stride, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return RLIS_ERR_UNSUPPORTED;
    sample_rows_kernel<<<rows, THREADS, 0, stream>>>(logits, params, out, vocab, row_stride);
    return RLIS_LAUNCH_CHECK();
}

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
constexpr int MAX_CHUNKS = 32;          // CTAs that share one row
constexpr int MAX_ROWS_CHUNKED = 4096;  // rows the chunked path has room for

// Scratch of the chunked path, part of the library image (no allocation, stable under CUDA graphs):
// the best (score, id) of every chunk, and a ticket counter per row that is zero between launches.
// Launches that overlap on the GPU (different streams) would race on it; the engine uses one stream.
__device__ float g_best_score[MAX_ROWS_CHUNKED * MAX_CHUNKS];
__device__ int g_best_id[MAX_ROWS_CHUNKED * MAX_CHUNKS];
__device__ int g_row_tickets[MAX_ROWS_CHUNKED];

__device__ __forceinline__ float row_score(float logit, int v, uint32_t key, float inv_t) {
    if (inv_t > 0.f) {
        const uint32_t h = lowbias32(key ^ ((uint32_t)v * 0x9e3779b9u));
        const float u = __fmul_rn((float)(h >> 9) + 0.5f, 1.0f / 8388608.0f);
        const float g = -logf(-logf(u));
        return __fadd_rn(__fmul_rn(logit, inv_t), g);
    }
    return logit;
}

// Best (score, id) over the block; valid in thread 0.
__device__ __forceinline__ void block_best(float& best, int& best_v, float* s_val, int* s_idx) {
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
    }
}

// grid (chunks, rows).  chunks == 1: the CTA scans the whole row.  Otherwise every CTA scans one
// chunk of the vocabulary and leaves its best in scratch; the CTA that takes the last ticket of
// the row (no CTA waits for another) folds the chunks in chunk order, so ties still go to the
// lowest id, and resets the ticket counter.
__global__ __launch_bounds__(THREADS) void sample_rows_kernel(const float* __restrict__ logits,
                                                              const uint32_t* __restrict__ params,
                                                              int* __restrict__ out, int vocab,
                                                              long long row_stride, int chunks) {
    pdl_wait();
    __shared__ float s_val[THREADS / 32];
    __shared__ int s_idx[THREADS / 32];
    __shared__ int s_last;
    const int r = blockIdx.y, ch = blockIdx.x;
    const float* row = logits + (size_t)r * row_stride;
    const uint32_t key = params[2 * r];
    const float inv_t = __uint_as_float(params[2 * r + 1]);
    const int per = (vocab + chunks - 1) / chunks;
    const int v0 = ch * per, v1 = min(v0 + per, vocab);
    float best = -INFINITY;
    int best_v = 0x7fffffff;
    for (int v = v0 + threadIdx.x; v < v1; v += THREADS) {
        const float s = row_score(row[v], v, key, inv_t);
        if (better(s, v, best, best_v)) { best = s; best_v = v; }
    }
    block_best(best, best_v, s_val, s_idx);
    if (chunks == 1) {
        // A row of NaNs or -inf leaves best_v at its sentinel: report id 0 as the reference's
        // argmax does (crates/engine/src/sampler.rs:238-246 starts from index 0).
        if (threadIdx.x == 0) out[r] = best_v == 0x7fffffff ? 0 : best_v;
        pdl_trigger();
        return;
    }
    if (threadIdx.x == 0) {
        g_best_score[r * MAX_CHUNKS + ch] = best;
        g_best_id[r * MAX_CHUNKS + ch] = best_v;
        __threadfence();
        s_last = atomicAdd(&g_row_tickets[r], 1) == chunks - 1;
    }
    __syncthreads();
    if (s_last && threadIdx.x == 0) {
        __threadfence();
        float bs = -INFINITY;
        int bv = 0x7fffffff;
        for (int i = 0; i < chunks; ++i) {
            const float os = __ldcg(&g_best_score[r * MAX_CHUNKS + i]);
            const int ov = __ldcg(&g_best_id[r * MAX_CHUNKS + i]);
            if (better(os, ov, bs, bv)) { bs = os; bv = ov; }
        }
        out[r] = bv == 0x7fffffff ? 0 : bv;
        g_row_tickets[r] = 0;
    }
    pdl_trigger();   // the next kernel of the stream may start its launch
}
}  // namespace

extern "C" int rlis_sample_rows(const float* logits, const uint32_t* params, int* out, int rows,
                                int vocab, long long row_stride, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return RLIS_ERR_UNSUPPORTED;
    int chunks = 1;
    if (rows <= MAX_ROWS_CHUNKED && rows < 128) {        // few rows: spread each over several CTAs
        chunks = (vocab + 4095) / 4096;
        if (chunks > MAX_CHUNKS) chunks = MAX_CHUNKS;
        if (chunks < 1) chunks = 1;
    }
    rlis_launch(sample_rows_kernel, dim3(chunks, rows), THREADS, 0, stream, logits, params, out, vocab, row_stride, chunks);
    return RLIS_LAUNCH_CHECK();
}

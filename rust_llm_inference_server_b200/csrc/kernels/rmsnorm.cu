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
    pdl_wait_and_trigger();
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

// The same for widths that are multiples of 4: 16-byte accesses, and the row is kept
// in registers between the sum of squares and the scaling (up to 4 vectors a thread).
template <typename T> struct Delta4;
template <> struct Delta4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Delta4<bf16> {
    static __device__ __forceinline__ float4 load(const bf16* p) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    static __device__ __forceinline__ void store(bf16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<uint32_t*>(&a);
        raw.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = raw;
    }
};

template <typename T>
__global__ void rmsnorm_vec4_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                    const float* __restrict__ w, T* __restrict__ out,
                                    const int* __restrict__ rows, int hidden, float eps) {
    __shared__ float scratch[33];
    constexpr int MAXV = 4;
    const size_t obase = (size_t)blockIdx.x * hidden;
    const size_t base = rows != nullptr ? (size_t)rows[blockIdx.x] * hidden : obase;
    const int nvec = hidden >> 2;
    float4 v[MAXV];
    pdl_wait_and_trigger();
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < MAXV; ++it) {
        const int i = it * blockDim.x + threadIdx.x;
        if (i < nvec) {
            float4 x = *reinterpret_cast<const float4*>(resid + base + 4 * (size_t)i);
            if (delta != nullptr) {
                const float4 dl = Delta4<T>::load(delta + base + 4 * (size_t)i);
                x.x += dl.x; x.y += dl.y; x.z += dl.z; x.w += dl.w;
                if (rows == nullptr) *reinterpret_cast<float4*>(resid + base + 4 * (size_t)i) = x;
            }
            v[it] = x;
            ss += x.x * x.x;
            ss += x.y * x.y;
            ss += x.z * x.z;
            ss += x.w * x.w;
        }
    }
    ss = block_sum(ss, scratch);
    const float rstd = 1.0f / sqrtf(ss / (float)hidden + eps);
#pragma unroll
    for (int it = 0; it < MAXV; ++it) {
        const int i = it * blockDim.x + threadIdx.x;
        if (i < nvec) {
            const float4 ww = *reinterpret_cast<const float4*>(w + 4 * (size_t)i);
            const float4 x = v[it];
            Delta4<T>::store(out + obase + 4 * (size_t)i,
                             make_float4(x.x * rstd * ww.x, x.y * rstd * ww.y, x.z * rstd * ww.z, x.w * rstd * ww.w));
        }
    }
}

extern "C" int rlis_rmsnorm(float* resid, const void* delta, const float* w, void* out,
                            const int* rows, int n_tokens, int hidden, float eps, int dtype,
                            cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    // many rows (portions of prompts): fewer threads with four vectors each keep more loads in
    // flight an SM (2048 rows of 2048: a 2048-token prefill of 16 layers 4.72 -> 4.64 ms)
    if (n_tokens > 64 && (hidden & 3) == 0) threads = min(threads, max(128, ((hidden + 15) / 16 + 31) / 32 * 32));
    if ((hidden & 3) == 0 && hidden <= threads * 16) {
        if (dtype == RLIS_F32)
            rlis_launch(rmsnorm_vec4_kernel<float>, n_tokens, threads, 0, stream, resid, (const float*)delta, w, (float*)out, rows, hidden, eps);
        else if (dtype == RLIS_BF16)
            rlis_launch(rmsnorm_vec4_kernel<bf16>, n_tokens, threads, 0, stream, resid, (const bf16*)delta, w, (bf16*)out, rows, hidden, eps);
        else
            return RLIS_ERR_UNSUPPORTED;
        return RLIS_LAUNCH_CHECK();
    }
    if (dtype == RLIS_F32)
        rlis_launch(rmsnorm_kernel<float>, n_tokens, threads, 0, stream, resid, (const float*)delta, w, (float*)out, rows, hidden, eps);
    else if (dtype == RLIS_BF16)
        rlis_launch(rmsnorm_kernel<bf16>, n_tokens, threads, 0, stream, resid, (const bf16*)delta, w, (bf16*)out, rows, hidden, eps);
    else
        return RLIS_ERR_UNSUPPORTED;
    return RLIS_LAUNCH_CHECK();
}

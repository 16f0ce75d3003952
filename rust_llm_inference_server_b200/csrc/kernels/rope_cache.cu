// Rotary position encoding of q and k, and the write of k and v into the paged cache, in one pass
// over the fused q|k|v projection output.
//
//   angle[j] = position * inv_freq[j]  (float32);  rotate-half:
//   out[j]       = x[j] cos - x[j + d/2] sin,   out[j + d/2] = x[j + d/2] cos + x[j] sin
// computed in float32 and rounded once (crates/model/src/rope.rs:61-78,111-117).  v is copied.
// Cache layout of one layer: [page, kv head, slot in page, d]; slot = table[pos / page] * page +
// pos % page is computed on the host (crates/model/src/paged.rs:258-263).  A negative slot means
// "do not store" (a call that reads another layer's cache).  inv_freq == nullptr: no rotation.
#include "common.cuh"

template <typename T>
__global__ void rope_cache_kernel(const T* __restrict__ qkv, T* __restrict__ q_out,
                                  T* __restrict__ k_cache, T* __restrict__ v_cache,
                                  const int* __restrict__ positions, const int* __restrict__ slots,
                                  const float* __restrict__ inv_freq, int nh, int nkv, int d,
                                  int page_size) {
    pdl_wait_and_trigger();
    extern __shared__ float cs[];  // cos[half], sin[half]
    const int t = blockIdx.x;
    const int half = d >> 1;
    float* c = cs;
    float* s = cs + half;
    const float pos = (float)positions[t];
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        if (inv_freq != nullptr) {
            float sn, cn;
            sincosf(pos * inv_freq[j], &sn, &cn);
            c[j] = cn;
            s[j] = sn;
        } else {
            c[j] = 1.f;
            s[j] = 0.f;
        }
    }
    __syncthreads();
    const int row_w = (nh + 2 * nkv) * d;
    const T* x = qkv + (size_t)t * row_w;
    const int slot = slots != nullptr ? slots[t] : -1;
    const long long page = slot >= 0 ? slot / page_size : 0;
    const int off = slot >= 0 ? slot % page_size : 0;
    const int n_pairs = (nh + 2 * nkv) * half;
    for (int idx = threadIdx.x; idx < n_pairs; idx += blockDim.x) {
        const int head = idx / half, j = idx - head * half;
        const float x1 = to_f<T>(x[head * d + j]);
        const float x2 = to_f<T>(x[head * d + j + half]);
        if (head < nh) {
            T* o = q_out + ((size_t)t * nh + head) * d;
            o[j] = from_f<T>(rope_first(x1, x2, c[j], s[j]));
            o[j + half] = from_f<T>(rope_second(x1, x2, c[j], s[j]));
        } else if (slot >= 0) {
            if (head < nh + nkv) {
                const int kvh = head - nh;
                T* o = k_cache + (((size_t)page * nkv + kvh) * page_size + off) * d;
                o[j] = from_f<T>(rope_first(x1, x2, c[j], s[j]));
                o[j + half] = from_f<T>(rope_second(x1, x2, c[j], s[j]));
            } else {
                const int kvh = head - nh - nkv;
                T* o = v_cache + (((size_t)page * nkv + kvh) * page_size + off) * d;
                o[j] = x[head * d + j];
                o[j + half] = x[head * d + j + half];
            }
        }
    }
}

// The same with 16-byte accesses: a thread takes one vector of the first half of a head and the
// matching vector of the second half (head sizes whose half is a multiple of the vector length).
template <typename T>
__global__ void rope_cache_vec_kernel(const T* __restrict__ qkv, T* __restrict__ q_out,
                                      T* __restrict__ k_cache, T* __restrict__ v_cache,
                                      const int* __restrict__ positions, const int* __restrict__ slots,
                                      const float* __restrict__ inv_freq, int nh, int nkv, int d,
                                      int page_size) {
    // Positions and slots are the step's own inputs, written before its first kernel: the angles
    // are ready by the time the projection before this kernel has finished.
    constexpr int VN = Vec16<T>::N;
    extern __shared__ float cs[];
    const int t = blockIdx.x;
    const int half = d >> 1;
    float* cc = cs;
    float* sn = cs + half;
    const float pos = (float)positions[t];
    const int slot = slots != nullptr ? slots[t] : -1;
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        float s_ = 0.f, c_ = 1.f;
        if (inv_freq != nullptr) sincosf(pos * inv_freq[j], &s_, &c_);
        cc[j] = c_;
        sn[j] = s_;
    }
    pdl_wait_and_trigger();
    __syncthreads();
    const T* x = qkv + (size_t)t * (nh + 2 * nkv) * d;
    const long long page = slot >= 0 ? slot / page_size : 0;
    const int off = slot >= 0 ? slot % page_size : 0;
    const int cph = half / VN;                       // vectors per half head
    const int items = (nh + 2 * nkv) * cph;
    for (int idx = threadIdx.x; idx < items; idx += blockDim.x) {
        const int head = idx / cph, j0 = (idx - head * cph) * VN;
        const uint4 r1 = *reinterpret_cast<const uint4*>(x + head * d + j0);
        const uint4 r2 = *reinterpret_cast<const uint4*>(x + head * d + half + j0);
        T* dst;
        if (head < nh) {
            dst = q_out + ((size_t)t * nh + head) * d;
        } else if (slot < 0) {
            continue;
        } else if (head < nh + nkv) {
            dst = k_cache + (((size_t)page * nkv + (head - nh)) * page_size + off) * d;
        } else {
            dst = v_cache + (((size_t)page * nkv + (head - nh - nkv)) * page_size + off) * d;
            *reinterpret_cast<uint4*>(dst + j0) = r1;
            *reinterpret_cast<uint4*>(dst + half + j0) = r2;
            continue;
        }
        float a[VN], b[VN];
        load16<T>(reinterpret_cast<const T*>(&r1), a);
        load16<T>(reinterpret_cast<const T*>(&r2), b);
        uint4 o1, o2;
        T* p1 = reinterpret_cast<T*>(&o1);
        T* p2 = reinterpret_cast<T*>(&o2);
#pragma unroll
        for (int e = 0; e < VN; ++e) {
            const float c_ = cc[j0 + e], s_ = sn[j0 + e];
            p1[e] = from_f<T>(rope_first(a[e], b[e], c_, s_));
            p2[e] = from_f<T>(rope_second(a[e], b[e], c_, s_));
        }
        *reinterpret_cast<uint4*>(dst + j0) = o1;
        *reinterpret_cast<uint4*>(dst + half + j0) = o2;
    }
}

extern "C" int rlis_rope_cache(const void* qkv, void* q_out, void* k_cache, void* v_cache,
                               const int* positions, const int* slots, const float* inv_freq,
                               int n_tokens, int nh, int nkv, int d, int page_size, int dtype,
                               cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (d <= 0 || (d & 1)) return RLIS_ERR_UNSUPPORTED;
    const int threads = 256;
    const size_t smem = (size_t)d * sizeof(float);
    const int vn = dtype == RLIS_F32 ? 4 : 8;
    if ((d / 2) % vn == 0 && (dtype == RLIS_F32 || dtype == RLIS_BF16)) {
        const int items = (nh + 2 * nkv) * (d / 2 / vn);
        const int th = items >= 256 ? 256 : (items >= 128 ? 128 : 64);
        if (dtype == RLIS_F32)
            rlis_launch(rope_cache_vec_kernel<float>, n_tokens, th, smem, stream, 
                (const float*)qkv, (float*)q_out, (float*)k_cache, (float*)v_cache, positions, slots, inv_freq,
                nh, nkv, d, page_size);
        else
            rlis_launch(rope_cache_vec_kernel<bf16>, n_tokens, th, smem, stream, 
                (const bf16*)qkv, (bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache, positions, slots, inv_freq,
                nh, nkv, d, page_size);
        return RLIS_LAUNCH_CHECK();
    }
    if (dtype == RLIS_F32)
        rlis_launch(rope_cache_kernel<float>, n_tokens, threads, smem, stream, 
            (const float*)qkv, (float*)q_out, (float*)k_cache, (float*)v_cache, positions, slots,
            inv_freq, nh, nkv, d, page_size);
    else if (dtype == RLIS_BF16)
        rlis_launch(rope_cache_kernel<bf16>, n_tokens, threads, smem, stream, 
            (const bf16*)qkv, (bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache, positions, slots,
            inv_freq, nh, nkv, d, page_size);
    else
        return RLIS_ERR_UNSUPPORTED;
    return RLIS_LAUNCH_CHECK();
}

// Token embedding lookup: one table row per token, widened into the float32 residual stream.
// Role in the reference: crates/model/src/layers.rs:199-204, llama.rs:256-262 (row select, no
// scaling by sqrt(hidden): `scale` is 1 there; a part may ask for another factor, applied in float32).
#include "common.cuh"

template <typename T>
__global__ void embedding_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                 float* __restrict__ out, int hidden, int vocab, float scale) {
    pdl_wait_and_trigger();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * hidden;
    if (id < 0 || id >= vocab) {  // the host rejects such ids before the launch; never read outside
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = 0.f;
        return;
    }
    const T* row = table + (size_t)id * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = to_f<T>(row[i]) * scale;
}

extern "C" int rlis_embedding(const int* ids, const void* table, float* out, int n_tokens,
                              int hidden, int vocab, float scale, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (dtype == RLIS_F32)
        rlis_launch(embedding_kernel<float>, n_tokens, threads, 0, stream, ids, (const float*)table, out, hidden, vocab, scale);
    else if (dtype == RLIS_BF16)
        rlis_launch(embedding_kernel<bf16>, n_tokens, threads, 0, stream, ids, (const bf16*)table, out, hidden, vocab, scale);
    else
        return RLIS_ERR_UNSUPPORTED;
    return RLIS_LAUNCH_CHECK();
}

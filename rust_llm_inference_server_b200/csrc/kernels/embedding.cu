// Token embedding lookup: one table row per token, widened into the float32 residual stream.
// Role in the reference: crates/model/src/layers.rs:199-204, llama.rs:256-262 (row select, no
// scaling by sqrt(hidden): `scale` is 1 there; a part may ask for another factor, applied in float32).
#include "common.cuh"
#include "mma_utils.cuh"

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

// The same lookup for a decode step whose first norm is taken apart (see stream_gemm_tcgen05.cu):
// beside the float32 row it writes xn = bf16(row * norm_weight) and, for every 128 features, the sum
// of the row's squares into partials[tile][token]; the product that follows applies
// 1 / sqrt(sum / hidden + eps).  A warp takes a tile of 128 features, four to a lane; hidden is a
// multiple of 4.
__global__ void embedding_sink_kernel(const int* __restrict__ ids, const bf16* __restrict__ table,
                                      float* __restrict__ out, const float* __restrict__ norm_weight,
                                      bf16* __restrict__ xn, float* __restrict__ partials, int n_tokens,
                                      int hidden, int vocab, float scale) {
    pdl_wait_and_trigger();
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool known = id >= 0 && id < vocab;    // the host rejects other ids before the launch; never read outside
    const bf16* row = table + (size_t)(known ? id : 0) * hidden;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int tiles = (hidden + 127) / 128;
    for (int tile = warp; tile < tiles; tile += warps) {
        const int f = tile * 128 + lane * 4;
        float ss = 0.f;
        if (f < hidden) {
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            if (known) {
                const uint2 raw = *reinterpret_cast<const uint2*>(row + f);
                const bf16* e = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
                for (int i = 0; i < 4; ++i) v[i] = __bfloat162float(e[i]) * scale;
            }
            const float4 w = *reinterpret_cast<const float4*>(norm_weight + f);
            *reinterpret_cast<float4*>(out + (size_t)t * hidden + f) = make_float4(v[0], v[1], v[2], v[3]);
            uint2 pk;
            pk.x = pack_bf16(v[0] * w.x, v[1] * w.y);
            pk.y = pack_bf16(v[2] * w.z, v[3] * w.w);
            *reinterpret_cast<uint2*>(xn + (size_t)t * hidden + f) = pk;
            ss = (v[0] * v[0] + v[1] * v[1]) + (v[2] * v[2] + v[3] * v[3]);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) partials[(size_t)tile * n_tokens + t] = ss;
    }
}

// out [n_tokens, hidden] float32, xn [n_tokens, hidden] bf16, partials [ceil(hidden / 128), n_tokens].
extern "C" int rlis_embedding_sink(const int* ids, const void* table, float* out, const float* norm_weight,
                                   void* xn, float* partials, int n_tokens, int hidden, int vocab, float scale,
                                   cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if ((hidden & 3) != 0) return RLIS_ERR_UNSUPPORTED;
    rlis_launch(embedding_sink_kernel, n_tokens, 128, 0, stream, ids, (const bf16*)table, out, norm_weight,
                (bf16*)xn, partials, n_tokens, hidden, vocab, scale);
    return RLIS_LAUNCH_CHECK();
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

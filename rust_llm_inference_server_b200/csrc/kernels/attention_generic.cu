// Causal grouped-query attention over the paged cache for any mix of query lengths: portions of
// prompts and single decoded tokens in one launch.  One warp per (token, query head).
//
// Query head h reads key/value head h / (nh / nkv) (crates/model/src/attention.rs:166-223).
// score = (q . k) * scale; keys after the query's position are hidden; with a window W > 0 keys at
// or before position - W are hidden too.  Scores, the running softmax and the p.v sum are float32
// (as in the reference's decode kernel, crates/model/src/paged_attention.rs:88-114).  Keys are
// taken in blocks of 32 that start at a multiple of 32, so the order of every sum depends only on
// the query's position: the same token gives the same bits however the batch was cut.
//
// With a token row list only those tokens of the step are computed (n_tokens = length of the list).
//
// This is the kernel of the float32 path and the fallback of the bfloat16 path for shapes that the
// tensor-core kernels refuse.  Head sizes: multiples of 16 up to 256.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int WARPS = 4;

template <typename T>
__global__ __launch_bounds__(WARPS * 32) void attn_generic_kernel(
    const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
    T* __restrict__ out, const int* __restrict__ seq_of_token, const int* __restrict__ positions,
    const int* __restrict__ block_tables, const int* __restrict__ token_rows, int max_blocks,
    int n_rows, int nh, int nkv, int d, int page_size, float scale, int window) {
    pdl_wait();
    extern __shared__ float qs_all[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gw = blockIdx.x * WARPS + warp;
    if (gw >= n_rows) return;  // no block-wide barrier below
    const int ti = gw / nh, h = gw - ti * nh;
    const int t = token_rows != nullptr ? token_rows[ti] : ti;   // a subset of the step's tokens
    const int kvh = h / (nh / nkv);
    const int pos = positions[t];
    const int* table = block_tables + (size_t)seq_of_token[t] * max_blocks;
    float* qs = qs_all + warp * d;
    const T* qrow = q + ((size_t)t * nh + h) * d;
    for (int j = lane; j < d; j += 32) qs[j] = to_f<T>(qrow[j]);
    __syncwarp();

    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    constexpr int VN = Vec16<T>::N;
    float m = -INFINITY, l = 0.f;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;

    for (int kb = lo - (lo & 31); kb <= pos; kb += 32) {
        const int key = kb + lane;
        const bool valid = key >= lo && key <= pos;
        float s = -INFINITY;
        // where this lane's key and value rows start (elements), or -1: hidden, or a page the host did not map
        long long row_off = -1;
        if (valid) {
            const int page = table[key / page_size];
            if (page < 0) {
                s = NAN;  // a page the host did not map: make it visible, never read outside
            } else {
                row_off = (((long long)page * nkv + kvh) * page_size + key % page_size) * d;
                const T* krow = k_cache + row_off;
                float dot = 0.f;
                for (int j = 0; j < d; j += VN) {
                    float kv[VN];
                    load16<T>(krow + j, kv);
#pragma unroll
                    for (int u = 0; u < VN; ++u) dot = fmaf(qs[j + u], kv[u], dot);
                }
                s = dot * scale;
            }
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = valid ? expf(s - m_new) : 0.f;
        const float corr = expf(m - m_new);
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] *= corr;
        // p . v in the order of the keys.  The rows' addresses come from the lanes that own the keys,
        // not from the table again, and a key without weight takes part with a zero that is selected,
        // not multiplied (its row may hold anything): no load waits for a branch, so the loads of
        // several keys are in flight together.
#pragma unroll 8
        for (int kk = 0; kk < 32; ++kk) {
            const float pk = __shfl_sync(0xffffffffu, p, kk);
            const long long off = __shfl_sync(0xffffffffu, row_off, kk);
            const bool use = pk != 0.f && off >= 0;  // uniform over the warp
            const T* vrow = v_cache + (use ? off : 0);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int dim = lane + 32 * i;
                if (dim < d) {
                    const float v = to_f<T>(vrow[dim]);
                    acc[i] = use ? fmaf(pk, v, acc[i]) : acc[i];
                }
            }
        }
        m = m_new;
    }
    T* orow = out + ((size_t)t * nh + h) * d;
    const float inv_l = 1.0f / l;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int dim = lane + 32 * i;
        if (dim < d) orow[dim] = from_f<T>(acc[i] * inv_l);
    }
    pdl_trigger();   // the next kernel of the stream may start its launch
}
}  // namespace

extern "C" int rlis_attention_generic(const void* q, const void* k_cache, const void* v_cache,
                                      void* out, const int* seq_of_token, const int* positions,
                                      const int* block_tables, const int* token_rows,
                                      int max_blocks, int n_tokens, int nh,
                                      int nkv, int d, int page_size, float scale, int window,
                                      int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (d % 16 != 0 || d > 256 || d <= 0 || nkv <= 0 || nh % nkv != 0) return RLIS_ERR_UNSUPPORTED;
    const long long n_rows = (long long)n_tokens * nh;
    if (n_rows > 0x7fffffffLL) return RLIS_ERR_UNSUPPORTED;
    const unsigned blocks = (unsigned)((n_rows + WARPS - 1) / WARPS);
    const size_t smem = (size_t)WARPS * d * sizeof(float);
    if (dtype == RLIS_F32)
        rlis_launch(attn_generic_kernel<float>, blocks, WARPS * 32, smem, stream, 
            (const float*)q, (const float*)k_cache, (const float*)v_cache, (float*)out, seq_of_token,
            positions, block_tables, token_rows, max_blocks, (int)n_rows, nh, nkv, d, page_size, scale, window);
    else if (dtype == RLIS_BF16)
        rlis_launch(attn_generic_kernel<bf16>, blocks, WARPS * 32, smem, stream, 
            (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out, seq_of_token,
            positions, block_tables, token_rows, max_blocks, (int)n_rows, nh, nkv, d, page_size, scale, window);
    else
        return RLIS_ERR_UNSUPPORTED;
    return RLIS_LAUNCH_CHECK();
}

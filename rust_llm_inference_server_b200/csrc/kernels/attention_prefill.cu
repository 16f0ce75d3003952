// Causal flash attention for portions of prompts over the paged cache (bfloat16, head sizes 64
// and 128): queries at positions P .. L-1 of a request, keys 0 .. L-1 read through its block
// table, the causal edge aligned to the end of the keys, as cutting prompts into portions needs.
//
// Role in the reference: the fused `sdpa` call for multi-token segments
// (crates/model/src/attention.rs:144-157), whose score matrix is never materialised, and the
// gather path's formulas (attention.rs:204-233): score = q.k * scale in float32, keys after the
// query hidden, softmax in float32.  The portion's own keys and values are already in the cache
// when this kernel runs (crates/model/src/paged.rs:336-337 stores before attending).
//
// One CTA = one query head x 64 tokens of one request (4 warps x 16 rows).  Key tiles of 64 are
// brought to shared memory by 16-byte asynchronous copies, double-buffered, rows padded by 8
// elements so that ldmatrix is free of bank conflicts.  Per tile and warp: S = Q K^T (m16n8k16,
// bf16 products, float32 sums), online softmax on S * scale, O += P V with P rounded to bf16 as
// the A operand and V through ldmatrix.trans.  Work items (request, first token of the tile) come
// from the host.  A window W > 0 also hides keys at or before position - W.
#include "common.cuh"
#include "mma_utils.cuh"
#include <math.h>

namespace {
constexpr int PF_WARPS = 4;
constexpr int PF_THREADS = PF_WARPS * 32;
constexpr int PF_BM = 64;   // query tokens per CTA
static_assert(PF_BM == RLIS_PREFILL_TILE, "the host's tile list is cut for another tile size");
constexpr int PF_BN = 64;   // keys per tile

template <int D>
__global__ __launch_bounds__(PF_THREADS) void attn_prefill_mma_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
    bf16* __restrict__ out, const int* __restrict__ tiles, const int* __restrict__ cu_seqlens,
    const int* __restrict__ ctx_lens, const int* __restrict__ block_tables, int max_blocks, int nh,
    int nkv, int page_size, float scale, int window) {
    pdl_wait();
    constexpr int STRIDE = D + 8;
    constexpr int KS = D / 16;
    constexpr int ND = D / 8;
    constexpr int CPR = D / 8;
    constexpr int TILE = PF_BN * STRIDE;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* sbase = reinterpret_cast<bf16*>(smem_raw);            // [stage][K|V][64][STRIDE]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, c = lane & 3;
    // x: the head, y: the tile; CTAs start in the order of the tile list across all heads
    const int b = tiles[2 * blockIdx.y], t0 = tiles[2 * blockIdx.y + 1];
    const int head = blockIdx.x;
    const int kvh = head / (nh / nkv);
    const int q_start = cu_seqlens[b];
    const int q_len = cu_seqlens[b + 1] - q_start;
    const int ctx = ctx_lens[b];
    const int start_pos = ctx - q_len;
    const int* table = block_tables + (size_t)b * max_blocks;
    const size_t head_stride = (size_t)page_size * D;

    // this lane's two rows: tokens t0 + warp*16 + g and + 8
    const int ti0 = t0 + warp * 16 + g, ti1 = ti0 + 8;
    const bool rv0 = ti0 < q_len, rv1 = ti1 < q_len;
    const int pos0 = start_pos + ti0, pos1 = start_pos + ti1;
    const int lo0 = window > 0 ? max(0, pos0 - window + 1) : 0;
    const int lo1 = window > 0 ? max(0, pos1 - window + 1) : 0;

    uint32_t qa[KS][4];
    {
        const bf16* q0 = q + ((size_t)(q_start + (rv0 ? ti0 : 0)) * nh + head) * D;
        const bf16* q1 = q + ((size_t)(q_start + (rv1 ? ti1 : 0)) * nh + head) * D;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            qa[ks][0] = rv0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 2 * c) : 0u;
            qa[ks][1] = rv1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 2 * c) : 0u;
            qa[ks][2] = rv0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 2 * c + 8) : 0u;
            qa[ks][3] = rv1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 2 * c + 8) : 0u;
        }
    }

    // keys this CTA can need: from the first row's window edge to the last row's position
    const int last_tok = min(t0 + PF_BM, q_len) - 1;
    const int k_hi = start_pos + last_tok + 1;                                  // exclusive
    const int k_lo = window > 0 ? max(0, start_pos + t0 - window + 1) : 0;
    const int kt0 = k_lo / PF_BN, kt1 = (k_hi + PF_BN - 1) / PF_BN;

    // (short address arithmetic: a power-of-two page size turns the division into a shift)
    const int page_shift = (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1;
    const size_t page_stride = (size_t)nkv * head_stride;
    const bf16* kbase = k_cache + (size_t)kvh * head_stride;
    const bf16* vbase = v_cache + (size_t)kvh * head_stride;
    const int key_in0 = threadIdx.x / CPR, c16 = threadIdx.x % CPR;
    constexpr int KEYS_PER_IT = PF_THREADS / CPR;
    const uint32_t sm_off0 = (uint32_t)(key_in0 * STRIDE + c16 * 8);
    auto issue = [&](int kt, int stage) {
        bf16* ks_ = sbase + (size_t)stage * 2 * TILE;
        bf16* vs_ = ks_ + TILE;
#pragma unroll
        for (int i = 0; i < (PF_BN * CPR) / PF_THREADS; ++i) {
            const int key = kt * PF_BN + key_in0 + i * KEYS_PER_IT;
            const bool valid = key < k_hi && key >= k_lo;
            size_t off = 0;
            if (valid) {
                const int pi = page_shift >= 0 ? key >> page_shift : key / page_size;
                const int in_page = page_shift >= 0 ? key & (page_size - 1) : key - pi * page_size;
                off = (size_t)table[pi] * page_stride + (uint32_t)(in_page * D + c16 * 8);
            }
            const uint32_t so = sm_off0 + (uint32_t)(i * KEYS_PER_IT * STRIDE);
            cp_async16(ks_ + so, kbase + off, valid);
            cp_async16(vs_ + so, vbase + off, valid);
        }
        cp_async_commit();
    };

    const float scale_log2 = scale * 1.4426950408889634f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float oacc[ND][4];
#pragma unroll
    for (int nd = 0; nd < ND; ++nd)
#pragma unroll
        for (int e = 0; e < 4; ++e) oacc[nd][e] = 0.f;

    int stage = 0;
    if (kt0 < kt1) issue(kt0, 0);
    for (int kt = kt0; kt < kt1; ++kt) {
        if (kt + 1 < kt1) {
            issue(kt + 1, stage ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const bf16* ks_ = sbase + (size_t)stage * 2 * TILE;
        const bf16* vs_ = ks_ + TILE;

        float sacc[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) sacc[nt][e] = 0.f;
#pragma unroll
            for (int ks2 = 0; ks2 < KS / 2; ++ks2) {
                uint32_t kb[4];
                ldmatrix_x4(kb, ks_ + (nt * 8 + (lane & 7)) * STRIDE + ks2 * 32 + (lane >> 3) * 8);
                mma_bf16_16816(sacc[nt], qa[2 * ks2], kb[0], kb[1]);
                mma_bf16_16816(sacc[nt], qa[2 * ks2 + 1], kb[2], kb[3]);
            }
        }
        // Scores in units of log2(e): s * scale * log2(e), so that exp(x) is one exp2 instruction
        // (softmax does not see the common factor).  Keys after the query (and before its window)
        // are hidden; tiles that lie wholly before every row's position skip the comparisons.
        const bool edge = (kt + 1) * PF_BN - 1 > start_pos + t0 + warp * 16 || window > 0;
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                float s0 = sacc[nt][e] * scale_log2, s1 = sacc[nt][2 + e] * scale_log2;
                if (edge) {
                    const int key = kt * PF_BN + nt * 8 + 2 * c + e;
                    if (!(key <= pos0 && key >= lo0)) s0 = -INFINITY;
                    if (!(key <= pos1 && key >= lo1)) s1 = -INFINITY;
                }
                sacc[nt][e] = s0;
                sacc[nt][2 + e] = s1;
                mx0 = fmaxf(mx0, s0);
                mx1 = fmaxf(mx1, s1);
            }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
        // a row that has seen no key yet (all hidden so far) keeps a zero state
        const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
        const float corr0 = exp2f(m_run[0] - ms0), corr1 = exp2f(m_run[1] - ms1);   // exp2(-inf) = 0
        float ls0 = 0.f, ls1 = 0.f;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const float p0 = exp2f(sacc[nt][e] - ms0), p1 = exp2f(sacc[nt][2 + e] - ms1);
                sacc[nt][e] = p0;
                sacc[nt][2 + e] = p1;
                ls0 += p0;
                ls1 += p1;
            }
        ls0 += __shfl_xor_sync(0xffffffffu, ls0, 1);
        ls0 += __shfl_xor_sync(0xffffffffu, ls0, 2);
        ls1 += __shfl_xor_sync(0xffffffffu, ls1, 1);
        ls1 += __shfl_xor_sync(0xffffffffu, ls1, 2);
        l_run[0] = l_run[0] * corr0 + ls0;
        l_run[1] = l_run[1] * corr1 + ls1;
        m_run[0] = mn0;
        m_run[1] = mn1;
#pragma unroll
        for (int nd = 0; nd < ND; ++nd) {
            oacc[nd][0] *= corr0;
            oacc[nd][1] *= corr0;
            oacc[nd][2] *= corr1;
            oacc[nd][3] *= corr1;
        }
#pragma unroll
        for (int kk = 0; kk < PF_BN / 16; ++kk) {
            uint32_t pa[4];
            pa[0] = pack_bf16(sacc[2 * kk][0], sacc[2 * kk][1]);
            pa[1] = pack_bf16(sacc[2 * kk][2], sacc[2 * kk][3]);
            pa[2] = pack_bf16(sacc[2 * kk + 1][0], sacc[2 * kk + 1][1]);
            pa[3] = pack_bf16(sacc[2 * kk + 1][2], sacc[2 * kk + 1][3]);
#pragma unroll
            for (int nd2 = 0; nd2 < ND / 2; ++nd2) {
                uint32_t vb[4];
                const int mat = lane >> 3;
                ldmatrix_x4_trans(vb, vs_ + (kk * 16 + (mat & 1) * 8 + (lane & 7)) * STRIDE + (nd2 * 2 + (mat >> 1)) * 8);
                mma_bf16_16816(oacc[2 * nd2], pa, vb[0], vb[1]);
                mma_bf16_16816(oacc[2 * nd2 + 1], pa, vb[2], vb[3]);
            }
        }
        __syncthreads();       // everyone is done with this stage before the next copies land in it
        stage ^= 1;
    }

    const float inv0 = l_run[0] > 0.f ? 1.0f / l_run[0] : 0.f;
    const float inv1 = l_run[1] > 0.f ? 1.0f / l_run[1] : 0.f;
    if (rv0) {
        bf16* o = out + ((size_t)(q_start + ti0) * nh + head) * D;
#pragma unroll
        for (int nd = 0; nd < ND; ++nd)
            *reinterpret_cast<uint32_t*>(o + nd * 8 + 2 * c) = pack_bf16(oacc[nd][0] * inv0, oacc[nd][1] * inv0);
    }
    if (rv1) {
        bf16* o = out + ((size_t)(q_start + ti1) * nh + head) * D;
#pragma unroll
        for (int nd = 0; nd < ND; ++nd)
            *reinterpret_cast<uint32_t*>(o + nd * 8 + 2 * c) = pack_bf16(oacc[nd][2] * inv1, oacc[nd][3] * inv1);
    }
    pdl_trigger();   // the next kernel of the stream may start its launch
}

template <int D> constexpr size_t prefill_smem_bytes() {
    return (size_t)2 * 2 * PF_BN * (D + 8) * sizeof(bf16);
}
}  // namespace

// tiles: int32 [n_tiles][2] = (batch entry, first token of the tile within the entry's portion);
// a tile covers 64 tokens.
extern "C" int rlis_attention_prefill(const void* q, const void* k_cache, const void* v_cache,
                                      void* out, const int* tiles, int n_tiles,
                                      const int* cu_seqlens, const int* ctx_lens,
                                      const int* block_tables, int max_blocks, int nh, int nkv,
                                      int d, int page_size, float scale, int window, int dtype,
                                      cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (dtype != RLIS_BF16 || (d != 64 && d != 128) || nkv <= 0 || nh % nkv != 0 || n_tiles > 65535)
        return RLIS_ERR_UNSUPPORTED;
    dim3 grid(nh, n_tiles);
    static bool attr_done = false;
    if (!attr_done) {
        cudaFuncSetAttribute(attn_prefill_mma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)prefill_smem_bytes<128>());
        attr_done = true;
    }
    if (d == 64)
        rlis_launch(attn_prefill_mma_kernel<64>, grid, PF_THREADS, prefill_smem_bytes<64>(), stream, 
            (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out, tiles, cu_seqlens, ctx_lens,
            block_tables, max_blocks, nh, nkv, page_size, scale, window);
    else
        rlis_launch(attn_prefill_mma_kernel<128>, grid, PF_THREADS, prefill_smem_bytes<128>(), stream, 
            (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out, tiles, cu_seqlens, ctx_lens,
            block_tables, max_blocks, nh, nkv, page_size, scale, window);
    return RLIS_LAUNCH_CHECK();
}

// Tokens a tile of the `tiles` list covers, for this kernel and for the tcgen05 one.
extern "C" int rlis_attention_prefill_tile(void) { return RLIS_PREFILL_TILE; }

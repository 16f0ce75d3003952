// Decode attention over the paged cache, split over the context: one query token per request,
// grid (kv head, request, split).  All query heads of a GQA group share every K and V row that the
// CTA reads, so the cache is streamed from HBM once per kv head.
//
// Role in the reference: the Metal kernels paged_attention_decode{,_split} and
// paged_attention_reduce (crates/model/src/paged_attention.metal:56-304) and their split plan
// (crates/model/src/paged_attention.rs:21-36): lanes take one key position each for q.k, an online
// softmax per block of positions, then lanes take slices of the head dimension for p.v; partial
// (m, l, acc) per split, merged afterwards.  Scores, softmax and p.v are float32; q.k accumulates
// over d in index order.
//
// Layout here: a warp owns blocks of 32 keys (strided over the CTA's 4 warps) and keeps its own
// running (m, l, acc); the four warps are merged through shared memory at the end, so the main
// loop has no block-wide barrier.  p.v: 8-element (16-byte) slices of a V row per lane.
//
// Scratch: when splits > 1 the kernel writes partial results [request, head, split, d + 2] float32
// to a caller-provided buffer and `attention_decode_combine` merges them.
#include "tcgen05_utils.cuh"
#include <math.h>

namespace {

constexpr int DEC_WARPS = 4;
constexpr int DEC_THREADS = DEC_WARPS * 32;

// NREP = query heads per kv head, D8 = head_dim / 8 (16-byte chunks per row).
template <int NREP>
__global__ __launch_bounds__(DEC_THREADS) void attn_decode_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
    bf16* __restrict__ out, float* __restrict__ partial, const int* __restrict__ dec_rows,
    const int* __restrict__ dec_seqs, const int* __restrict__ ctx_lens,
    const int* __restrict__ block_tables, int max_blocks, int nh, int nkv, int d, int page_size,
    float scale, int window, int splits) {
    pdl_wait_and_trigger();
    extern __shared__ __align__(16) float smem[];
    // smem: q [NREP][d] | p per warp [DEC_WARPS][32][NREP] | merge area
    float* qs = smem;
    float* ps = qs + NREP * d;
    float* merge = ps + DEC_WARPS * 32 * NREP;   // [DEC_WARPS][groups][NREP][d] then [DEC_WARPS][NREP][2]

    const int kvh = blockIdx.x, bi = blockIdx.y, split = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = dec_rows[bi];
    const int seq = dec_seqs[bi];
    const int ctx = ctx_lens[seq];          // keys 0 .. ctx-1; the query sits at ctx-1
    const int* table = block_tables + (size_t)seq * max_blocks;
    const int d8 = d >> 3;

    // this split's range of keys, in whole blocks of 32
    const int lo_all = window > 0 ? max(0, ctx - window) : 0;
    const int first_blk = lo_all >> 5;
    const int n_blk = ((ctx + 31) >> 5) - first_blk;
    const int blk_per_split = (n_blk + splits - 1) / splits;
    const int blk0 = first_blk + split * blk_per_split;
    const int blk1 = min(blk0 + blk_per_split, first_blk + n_blk);

    for (int i = threadIdx.x; i < NREP * d; i += DEC_THREADS) {
        const int h = i / d, j = i - h * d;
        qs[i] = to_f<bf16>(q[((size_t)row * nh + kvh * NREP + h) * d + j]);
    }
    __syncthreads();

    float m[NREP], l[NREP];
    float acc[NREP][8];
#pragma unroll
    for (int h = 0; h < NREP; ++h) {
        m[h] = -INFINITY;
        l[h] = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[h][e] = 0.f;
    }
    // p.v mapping: lane -> (key within a group, 16-byte chunk of the row)
    const int kpi = 32 / d8 > 0 ? 32 / d8 : 1;          // keys per iteration of a warp (d8 <= 32)
    const int pv_key = lane / d8, pv_chunk = lane - pv_key * d8;
    const bool pv_active = lane < kpi * d8;
    float* pw = ps + warp * 32 * NREP;

    for (int blk = blk0 + warp; blk < blk1; blk += DEC_WARPS) {
        const int key = (blk << 5) + lane;
        const bool valid = key >= lo_all && key < ctx;
        float s[NREP];
#pragma unroll
        for (int h = 0; h < NREP; ++h) s[h] = -INFINITY;
        if (valid) {
            const int page = table[key / page_size];
            const bf16* krow = k_cache + (((size_t)page * nkv + kvh) * page_size + key % page_size) * d;
#pragma unroll
            for (int h = 0; h < NREP; ++h) s[h] = 0.f;
            for (int c = 0; c < d8; ++c) {
                float kf[8];
                load16<bf16>(krow + c * 8, kf);
#pragma unroll
                for (int h = 0; h < NREP; ++h) {
                    const float4 qa = *reinterpret_cast<const float4*>(qs + h * d + c * 8);
                    const float4 qb = *reinterpret_cast<const float4*>(qs + h * d + c * 8 + 4);
                    float t = s[h];
                    t = fmaf(qa.x, kf[0], t); t = fmaf(qa.y, kf[1], t);
                    t = fmaf(qa.z, kf[2], t); t = fmaf(qa.w, kf[3], t);
                    t = fmaf(qb.x, kf[4], t); t = fmaf(qb.y, kf[5], t);
                    t = fmaf(qb.z, kf[6], t); t = fmaf(qb.w, kf[7], t);
                    s[h] = t;
                }
            }
#pragma unroll
            for (int h = 0; h < NREP; ++h) s[h] *= scale;
        }
        float corr[NREP];
#pragma unroll
        for (int h = 0; h < NREP; ++h) {
            const float m_new = fmaxf(m[h], warp_max(s[h]));   // finite: every block has a valid key
            const float p = valid ? expf(s[h] - m_new) : 0.f;
            corr[h] = expf(m[h] - m_new);
            l[h] = l[h] * corr[h] + warp_sum(p);
            m[h] = m_new;
            pw[lane * NREP + h] = p;
        }
        __syncwarp();
#pragma unroll
        for (int h = 0; h < NREP; ++h)
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[h][e] *= corr[h];
        if (pv_active) {
            for (int k0 = 0; k0 < 32; k0 += kpi) {
                const int kk = k0 + pv_key;
                const int kidx = (blk << 5) + kk;
                if (kk < 32 && kidx >= lo_all && kidx < ctx) {
                    const int page = table[kidx / page_size];
                    const bf16* vrow = v_cache + (((size_t)page * nkv + kvh) * page_size + kidx % page_size) * d;
                    float vf[8];
                    load16<bf16>(vrow + pv_chunk * 8, vf);
#pragma unroll
                    for (int h = 0; h < NREP; ++h) {
                        const float p = pw[kk * NREP + h];
#pragma unroll
                        for (int e = 0; e < 8; ++e) acc[h][e] = fmaf(p, vf[e], acc[h][e]);
                    }
                }
            }
        }
        __syncwarp();
    }

    // Per-warp results to shared memory.  Lanes with the same chunk but another key group hold
    // partial sums over different keys: each group writes its own copy, summed below in a fixed
    // order.  stage[warp][group][h][d]; ml[warp][h][2].
    const int groups = kpi;
    float* stage = merge + (size_t)warp * groups * NREP * d;
    if (pv_active) {
#pragma unroll
        for (int h = 0; h < NREP; ++h)
#pragma unroll
            for (int e = 0; e < 8; ++e) stage[((size_t)pv_key * NREP + h) * d + pv_chunk * 8 + e] = acc[h][e];
    }
    float* ml = merge + (size_t)DEC_WARPS * groups * NREP * d;
    if (lane == 0) {
#pragma unroll
        for (int h = 0; h < NREP; ++h) {
            ml[(warp * NREP + h) * 2] = m[h];
            ml[(warp * NREP + h) * 2 + 1] = l[h];
        }
    }
    __syncthreads();

    // merge the warps: big = max m; out = sum acc_w * exp(m_w - big) / sum l_w * exp(m_w - big)
    for (int i = threadIdx.x; i < NREP * d; i += DEC_THREADS) {
        const int h = i / d, j = i - h * d;
        float big = -INFINITY;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) big = fmaxf(big, ml[(w * NREP + h) * 2]);
        float a = 0.f, lsum = 0.f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) {
            const float mw = ml[(w * NREP + h) * 2];
            if (mw == -INFINITY) continue;          // this warp had no block of keys
            const float wgt = expf(mw - big);
            float aw = 0.f;
            for (int g = 0; g < groups; ++g) aw += merge[(((size_t)w * groups + g) * NREP + h) * d + j];
            a += aw * wgt;
            lsum += ml[(w * NREP + h) * 2 + 1] * wgt;
        }
        const int head = kvh * NREP + h;
        if (splits == 1) {
            out[((size_t)row * nh + head) * d + j] = from_f<bf16>(a / lsum);
        } else {
            float* pr = partial + (((size_t)bi * nh + head) * splits + split) * (d + 2);
            pr[j] = a;
            if (j == 0) {
                pr[d] = big;
                pr[d + 1] = lsum;
            }
        }
    }
}

// Tensor-core version for head sizes 64 and 128 (groups of up to 8 query heads).  The CUDA-core
// kernel above needs about 750 lane-instructions per key and kv head, which caps it near a fifth of
// the HBM rate; here the heads of a group are the rows of an m16n8k16 tile, so a key costs a few
// tensor instructions and the kernel waits on memory only.
//
// Per warp: blocks of 32 keys in a ring of 2 to 4 stages in shared memory.  Head size 64 (TMA):
// a block is one to four bulk tensor copies of the cache seen as a [rows, 64] tensor (a page, or 32
// rows of one), 128-byte swizzle, an mbarrier per stage and warp; ldmatrix XORs the 16-byte chunk
// index with the row's index in its group of 8.  Otherwise 16-byte asynchronous copies into rows
// padded to D + 8 elements.  (The 16-byte copies stopped at 4.9 TB/s with 96 KB in flight an SM,
// and more stages did not help them; the bulk copies reach 5.65 TB/s at batch 64 and take 14.2
// instead of 17.4 us at batch 8.)
//   S[heads x 32 keys] = Q K^T      (K rows through ldmatrix, bf16 products, float32 sums)
//   online softmax in float32 on S * scale
//   O[heads x D]      += P V        (P rounded to bf16 as the A operand, V through ldmatrix.trans)
// With `qkv` set the kernel does the work of the rotation kernel too, for steps that decode only:
// q comes straight from the q|k|v projection and is rotated as it is loaded; the warp that meets
// the block with the request's newest key rotates that key, puts key and value into its tile and
// into the cache (slots == nullptr: the layer reads another layer's cache and stores nothing).
// The arithmetic is that of rope_cache.cu, bit for bit.
struct DecodeQkv {
    const bf16* qkv;            // [tokens, (nh + 2 nkv) d], or nullptr: q is rotated and the cache is written already
    const int* positions;       // [tokens]
    const int* slots;           // [tokens] page * page_size + offset of the token's key, or nullptr
    const float* inv_freq;      // [d / 2], or nullptr: no rotation
    bf16* k_cache;              // the same arrays as the kernel reads, for the newest key
    bf16* v_cache;
};

constexpr int DEC_TABLE_SLOTS = 512;      // block-table entries of a CTA kept in shared memory (2 KB: three CTAs of head size 64 still fit an SM)


template <int D, int NSTAGE, bool TMA>
__global__ __launch_bounds__(DEC_THREADS) void attn_decode_mma_kernel(
    const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, int cache_rows,
    const bf16* __restrict__ q, const bf16* k_cache, const bf16* v_cache,
    bf16* __restrict__ out, float* __restrict__ partial, const int* __restrict__ dec_rows,
    const int* __restrict__ dec_seqs, const int* __restrict__ ctx_lens,
    const int* __restrict__ block_tables, int max_blocks, int nh, int nkv, int nrep, int page_size,
    float scale, int window, int splits, int* __restrict__ tickets, DecodeQkv fz, int cluster_merge) {
    __shared__ int s_last;
    __shared__ float s_cos[D / 2], s_sin[D / 2];
    __shared__ int s_table[DEC_TABLE_SLOTS];
    __shared__ uint64_t s_full[DEC_WARPS][NSTAGE];     // TMA: a stage of a warp has arrived
    __shared__ int s_abort;
    // TMA: a tile of 32 rows is D / 64 sub-tiles of [32 rows][64 elements]: rows of 128 bytes under the
    // 128-byte swizzle instead of padded rows (head size 128: the two halves of a row lie 4 KB apart)
    constexpr int STRIDE = TMA ? D : D + 8;  // elements per row (padded rows; for the tile's size)
    constexpr int HALVES = D / 64;           // TMA: sub-tiles of a tile
    // element offset, within a K or V tile, of the 16-byte chunk `chunk` of row r
    auto tile_off = [](int r, int chunk) -> int {
        return TMA ? (chunk >> 3) * (32 * 64) + r * 64 + (((chunk & 7) ^ (r & 7)) << 3) : r * STRIDE + (chunk << 3);
    };
    constexpr int KS = D / 16;               // k-steps of Q K^T
    constexpr int ND = D / 8;                // n-tiles of P V
    constexpr int CPR = D / 8;               // 16-byte chunks per row
    constexpr int TILE = 32 * STRIDE;        // elements of one K or V tile
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, c = lane & 3;
    bf16* wbase = reinterpret_cast<bf16*>(smem_raw) + (size_t)warp * NSTAGE * 2 * TILE;   // [stage][K|V][32][STRIDE]
    if (TMA) {
        if ((smem_u32(smem_raw) & 1023u) != 0u) {      // the swizzled tiles need it; checked, never seen
            if (threadIdx.x == 0) atomicExch(&tc::g_tc_error, 2);
            return;
        }
        if (threadIdx.x == 0) s_abort = 0;
        if (lane == 0) {
            for (int i = 0; i < NSTAGE; ++i) tc::bar_init(&s_full[warp][i], 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncthreads();
    }

    const int kvh = blockIdx.x, bi = blockIdx.y, split = blockIdx.z;
    const int row = dec_rows[bi];
    const int seq = dec_seqs[bi];
    const int ctx = ctx_lens[seq];
    const int* table = block_tables + (size_t)seq * max_blocks;
    const int lo_all = window > 0 ? max(0, ctx - window) : 0;
    const int first_blk = lo_all >> 5;
    const int n_blk = ((ctx + 31) >> 5) - first_blk;
    const int blk_per_split = (n_blk + splits - 1) / splits;
    const int blk0 = first_blk + split * blk_per_split;
    const int blk1 = min(blk0 + blk_per_split, first_blk + n_blk);
    const size_t head_stride = (size_t)page_size * D;

    // Address arithmetic of the copies is kept short: it runs 2 * CPR times per block and lane and
    // would otherwise outweigh the tensor work.  A page size that is a power of two (the usual
    // case) turns the division into a shift.
    const int page_shift = (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1;
    const size_t page_stride = (size_t)nkv * head_stride;
    const bf16* kbase = k_cache + (size_t)kvh * head_stride;
    const bf16* vbase = v_cache + (size_t)kvh * head_stride;
    // This CTA's part of the block table, fetched once (it is an input of the step): a lookup in
    // global memory per copy would sit on the path of every request for keys.
    const int page0 = page_shift >= 0 ? (blk0 << 5) >> page_shift : (blk0 << 5) / page_size;
    const int key_end = min(blk1 << 5, ctx);
    const int n_pages = key_end > (blk0 << 5) ? (page_shift >= 0 ? (key_end - 1) >> page_shift : (key_end - 1) / page_size) - page0 + 1 : 0;
    const bool table_in_smem = n_pages <= DEC_TABLE_SLOTS;
    if (table_in_smem) {
        for (int i = threadIdx.x; i < n_pages; i += DEC_THREADS) s_table[i] = table[page0 + i];
        __syncthreads();
    }
    const int key_in0 = lane / CPR, c16 = lane % CPR;       // chunk i of a lane: key_in0 + i * (32 / CPR)
    const uint32_t sm_off0 = (uint32_t)(key_in0 * STRIDE + c16 * 8);
    // TMA: a block of 32 keys is 32 / min(page, 32) boxes (times D / 64 column halves) of the cache
    // seen as [rows, D]; a box wholly past the context or behind the window is asked for past the end
    // of the tensor and arrives as zeros.  One lane announces the bytes, then a lane per box issues
    // its copy.
    const int box_rows = page_size < 32 ? page_size : 32;
    const int boxes = 32 / box_rows;
    auto issue = [&](int blk, int stage) {
        bf16* ks_ = wbase + (size_t)stage * 2 * TILE;
        bf16* vs_ = ks_ + TILE;
        if (TMA) {
            // the tile was read by ldmatrix until a moment ago: order those reads before the copy
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) tc::bar_expect_tx(&s_full[warp][stage], 2 * 32 * D * 2);
            __syncwarp();
            if (lane < 2 * boxes * HALVES) {
                const int bx = lane % boxes;
                const int half = (lane / boxes) % HALVES;
                const bool is_v = lane >= boxes * HALVES;
                const int key = (blk << 5) + bx * box_rows;
                const bool wanted = key < ctx && key + box_rows > lo_all;
                int rowc = cache_rows;
                if (wanted) {
                    const int pi = page_shift >= 0 ? key >> page_shift : key / page_size;
                    const int in_page = page_shift >= 0 ? key & (page_size - 1) : key - pi * page_size;
                    const int page = table_in_smem ? s_table[pi - page0] : table[pi];
                    rowc = (page * nkv + kvh) * page_size + in_page;
                }
                tc::tma_load_2d((is_v ? vs_ : ks_) + half * (32 * 64) + bx * box_rows * 64, is_v ? &map_v : &map_k,
                                half * 64, rowc, &s_full[warp][stage]);
            }
        } else {
#pragma unroll
        for (int i = 0; i < CPR; ++i) {               // 32 * CPR chunks, 32 lanes
            const int key_in = key_in0 + i * (32 / CPR);
            const int key = (blk << 5) + key_in;
            const bool valid = key >= lo_all && key < ctx;
            size_t off = 0;
            if (valid) {
                const int pi = page_shift >= 0 ? key >> page_shift : key / page_size;
                const int in_page = page_shift >= 0 ? key & (page_size - 1) : key - pi * page_size;
                const int page = table_in_smem ? s_table[pi - page0] : table[pi];
                off = (size_t)page * page_stride + (uint32_t)(in_page * D + c16 * 8);
            }
            const uint32_t so = sm_off0 + (uint32_t)(i * (32 / CPR) * STRIDE);
            cp_async16(ks_ + so, kbase + off, valid);
            cp_async16(vs_ + so, vbase + off, valid);
        }
        cp_async_commit();
        }
    };

    // scores are kept in units of log2(e) (s * scale * log2 e): exp becomes a single exp2
    const float scale_log2 = scale * 1.4426950408889634f;
    float m_run = -INFINITY, l_run = 0.f;      // of row g (every lane of a quad holds a copy)
    float oacc[ND][4];
#pragma unroll
    for (int nd = 0; nd < ND; ++nd)
#pragma unroll
        for (int e = 0; e < 4; ++e) oacc[nd][e] = 0.f;

    // NSTAGE - 1 blocks are in flight while one is worked on; a group is committed every turn
    // (an empty one past the end), so that "all but the newest NSTAGE - 1 groups" is always the
    // block that is needed.
    // The step's own inputs (rows, lengths, block tables) were written before its first kernel,
    // and of this layer's cache the kernel before this one (rotation and cache write) writes only
    // each request's newest key, ctx - 1.  So blocks that end before that key are requested before
    // this kernel waits for its predecessor; the block that holds it, and q, after.
    int blk = blk0 + warp;
    int stage = 0;
    const int newest_blk = (ctx - 1) >> 5;
    const bool fused = fz.qkv != nullptr;
    if (fused) {                // the angles of this token: positions are an input of the step
        const float pos = (float)fz.positions[row];
        for (int j = threadIdx.x; j < D / 2; j += DEC_THREADS) {
            float sn = 0.f, cn = 1.f;
            if (fz.inv_freq != nullptr) sincosf(pos * fz.inv_freq[j], &sn, &cn);
            s_cos[j] = cn;
            s_sin[j] = sn;
        }
    }
    int deferred_from = NSTAGE - 1;
#pragma unroll
    for (int i = 0; i < NSTAGE - 1; ++i) {
        const int b = blk + i * DEC_WARPS;
        if (b < blk1 && b < newest_blk && deferred_from == NSTAGE - 1) issue(b, i);
        else if (deferred_from == NSTAGE - 1) deferred_from = i;
    }
    pdl_wait_and_trigger();
#pragma unroll
    for (int i = 0; i < NSTAGE - 1; ++i) {
        if (i < deferred_from) continue;
        const int b = blk + i * DEC_WARPS;
        if (b < blk1) issue(b, i);
        else if (!TMA) cp_async_commit();
    }

    // Q as A fragments: row g = head g of the group (rows >= nrep and rows 8..15 are zero)
    uint32_t qa[KS][4];
    if (!fused) {
        const bf16* qrow = q + ((size_t)row * nh + kvh * nrep + (g < nrep ? g : 0)) * D;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            qa[ks][0] = g < nrep ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * c) : 0u;
            qa[ks][1] = 0u;
            qa[ks][2] = g < nrep ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * c + 8) : 0u;
            qa[ks][3] = 0u;
        }
    } else {
        __syncthreads();        // the angles
        const bf16* qrow = fz.qkv + (size_t)row * (nh + 2 * nkv) * D + (size_t)(kvh * nrep + (g < nrep ? g : 0)) * D;
        auto rotated = [&](int d0) -> uint32_t {      // dims d0, d0 + 1 of the rotated head, packed
            const bool first = d0 < D / 2;
            const int j = first ? d0 : d0 - D / 2;
            const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(qrow + j);
            const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(qrow + j + D / 2);
            const float a0 = __bfloat162float(lo.x), a1 = __bfloat162float(lo.y);
            const float b0 = __bfloat162float(hi.x), b1 = __bfloat162float(hi.y);
            return first ? pack_bf16(rope_first(a0, b0, s_cos[j], s_sin[j]), rope_first(a1, b1, s_cos[j + 1], s_sin[j + 1]))
                         : pack_bf16(rope_second(a0, b0, s_cos[j], s_sin[j]), rope_second(a1, b1, s_cos[j + 1], s_sin[j + 1]));
        };
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            qa[ks][0] = g < nrep ? rotated(ks * 16 + 2 * c) : 0u;
            qa[ks][1] = 0u;
            qa[ks][2] = g < nrep ? rotated(ks * 16 + 2 * c + 8) : 0u;
            qa[ks][3] = 0u;
        }
    }

    int turn = 0;                              // blocks this warp has worked on: block i sits in stage i % NSTAGE
    bool arrived = true;
    while (blk < blk1) {
        const int nblk = blk + DEC_WARPS;
        {
            const int ahead = blk + (NSTAGE - 1) * DEC_WARPS;
            const int st = stage == 0 ? NSTAGE - 1 : stage - 1;       // the stage worked on last turn
            if (ahead < blk1) issue(ahead, st);
            else if (!TMA) cp_async_commit();
            if (TMA) arrived = tc::bar_wait(&s_full[warp][stage], (uint32_t)(turn / NSTAGE) & 1u, &s_abort) && arrived;
            else cp_async_wait<NSTAGE - 1>();
        }
        ++turn;
        __syncwarp();
        const bf16* ks_ = wbase + (size_t)stage * 2 * TILE;
        const bf16* vs_ = ks_ + TILE;
        if (TMA && (blk << 5) + 31 >= ctx) {
            // slots of the last page past the context hold whatever was there before; a zero of P
            // times a NaN would still be a NaN: those rows of V are cleared (a lane per row)
            if ((blk << 5) + lane >= ctx) {
#pragma unroll
                for (int hf = 0; hf < HALVES; ++hf) {
                    uint4* vr = reinterpret_cast<uint4*>(const_cast<bf16*>(vs_) + hf * (32 * 64) + lane * 64);
#pragma unroll
                    for (int i = 0; i < 8; ++i) vr[i] = make_uint4(0u, 0u, 0u, 0u);
                }
            }
            __syncwarp();
        }
        if (fused && fz.slots != nullptr && blk == newest_blk) {
            // the request's newest key and value: from the projection into this tile and into the cache
            const int r = (ctx - 1) & 31;
            const bf16* krow = fz.qkv + (size_t)row * (nh + 2 * nkv) * D + (size_t)(nh + kvh) * D;
            const bf16* vrow = krow + (size_t)nkv * D;
            const int slot = fz.slots[row];
            if (slot >= 0) {
            const size_t at = (((size_t)(slot / page_size) * nkv + kvh) * page_size + (size_t)(slot % page_size)) * D;
            bf16* kt = const_cast<bf16*>(ks_);
            bf16* vt = const_cast<bf16*>(vs_);
            // where element j of row r sits (with the swizzle, its 16-byte chunk is XORed with r % 8)
            auto at_el = [&](int j) { return tile_off(r, j >> 3) | (j & 7); };
            for (int j = lane; j < D / 2; j += 32) {
                const float a = __bfloat162float(krow[j]), b = __bfloat162float(krow[j + D / 2]);
                const bf16 k1 = from_f<bf16>(rope_first(a, b, s_cos[j], s_sin[j]));
                const bf16 k2 = from_f<bf16>(rope_second(a, b, s_cos[j], s_sin[j]));
                const bf16 v1 = vrow[j], v2 = vrow[j + D / 2];
                kt[at_el(j)] = k1;
                kt[at_el(j + D / 2)] = k2;
                vt[at_el(j)] = v1;
                vt[at_el(j + D / 2)] = v2;
                fz.k_cache[at + j] = k1;
                fz.k_cache[at + j + D / 2] = k2;
                fz.v_cache[at + j] = v1;
                fz.v_cache[at + j + D / 2] = v2;
            }
            }
            __syncwarp();
        }

        float sacc[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) sacc[nt][e] = 0.f;
#pragma unroll
            for (int ks2 = 0; ks2 < KS / 2; ++ks2) {
                uint32_t kb[4];
                // (swizzle: the 16-byte chunk index is XORed with the row's index in its group of 8)
                const int kchunk = ks2 * 4 + (lane >> 3);
                ldmatrix_x4(kb, ks_ + tile_off(nt * 8 + (lane & 7), kchunk));
                mma_bf16_16816(sacc[nt], qa[2 * ks2], kb[0], kb[1]);
                mma_bf16_16816(sacc[nt], qa[2 * ks2 + 1], kb[2], kb[3]);
            }
        }
        // softmax over this block for row g
        float p[4][2];
        float mx = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = (blk << 5) + nt * 8 + 2 * c + e;
                const float sv = (key >= lo_all && key < ctx) ? sacc[nt][e] * scale_log2 : -INFINITY;
                p[nt][e] = sv;
                mx = fmaxf(mx, sv);
            }
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx);          // finite: every block holds a visible key
        const float corr = exp2f(m_run - m_new);
        float lsum = 0.f;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                p[nt][e] = exp2f(p[nt][e] - m_new);
                lsum += p[nt][e];
            }
        lsum += __shfl_xor_sync(0xffffffffu, lsum, 1);
        lsum += __shfl_xor_sync(0xffffffffu, lsum, 2);
        l_run = l_run * corr + lsum;
        m_run = m_new;
#pragma unroll
        for (int nd = 0; nd < ND; ++nd) {
            oacc[nd][0] *= corr;
            oacc[nd][1] *= corr;
        }
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
            uint32_t pa[4];
            pa[0] = pack_bf16(p[2 * kk][0], p[2 * kk][1]);
            pa[1] = 0u;
            pa[2] = pack_bf16(p[2 * kk + 1][0], p[2 * kk + 1][1]);
            pa[3] = 0u;
#pragma unroll
            for (int nd2 = 0; nd2 < ND / 2; ++nd2) {
                uint32_t vb[4];
                const int mat = lane >> 3;
                const int vchunk = nd2 * 2 + (mat >> 1);
                ldmatrix_x4_trans(vb, vs_ + tile_off(kk * 16 + (mat & 1) * 8 + (lane & 7), vchunk));
                mma_bf16_16816(oacc[2 * nd2], pa, vb[0], vb[1]);
                mma_bf16_16816(oacc[2 * nd2 + 1], pa, vb[2], vb[3]);
            }
        }
        __syncwarp();                                   // the stage may be overwritten from here on
        blk = nblk;
        stage = stage + 1 == NSTAGE ? 0 : stage + 1;
    }

    // merge the warps through shared memory (the tiles are no longer needed)
    __syncthreads();
    float* merge = reinterpret_cast<float*>(smem_raw);          // [DEC_WARPS][nrep][D]
    float* ml = merge + (size_t)DEC_WARPS * nrep * D;           // [DEC_WARPS][nrep][2]
    if (g < nrep) {
        float* mo = merge + ((size_t)warp * nrep + g) * D;
#pragma unroll
        for (int nd = 0; nd < ND; ++nd) {
            mo[nd * 8 + 2 * c] = oacc[nd][0];
            mo[nd * 8 + 2 * c + 1] = oacc[nd][1];
        }
        if (c == 0) {
            ml[(warp * nrep + g) * 2] = m_run;
            ml[(warp * nrep + g) * 2 + 1] = l_run;
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nrep * D; i += DEC_THREADS) {
        const int h = i / D, j = i - h * D;
        float big = -INFINITY;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) big = fmaxf(big, ml[(w * nrep + h) * 2]);
        float a = 0.f, lsum = 0.f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) {
            const float mw = ml[(w * nrep + h) * 2];
            if (mw == -INFINITY) continue;              // this warp had no block of keys
            const float wgt = exp2f(mw - big);
            a += merge[((size_t)w * nrep + h) * D + j] * wgt;
            lsum += ml[(w * nrep + h) * 2 + 1] * wgt;
        }
        const int head = kvh * nrep + h;
        if (splits == 1) {
            out[((size_t)row * nh + head) * D + j] = from_f<bf16>(a / lsum);
        } else if (cluster_merge) {
            float* cl = ml + DEC_WARPS * nrep * 2;          // [nrep][D], then m [nrep], l [nrep]
            cl[i] = a;
            if (j == 0) {
                cl[nrep * D + h] = big * 0.6931471805599453f;
                cl[nrep * D + nrep + h] = lsum;
            }
        } else {
            float* pr = partial + (((size_t)bi * nh + head) * splits + split) * (D + 2);
            pr[j] = a;
            if (j == 0) {
                pr[D] = big * 0.6931471805599453f;      // back to natural units, as the merge reads it
                pr[D + 1] = lsum;
            }
        }
    }
    if (splits > 1 && cluster_merge) {
        // The splits of a (request, kv head) are the CTAs of a cluster: each has left its sums in
        // its own shared memory, and after the barrier CTA r merges a slice of the outputs from all
        // of them through distributed shared memory, in split order.  No trip through global memory.
        const float* cl = ml + DEC_WARPS * nrep * 2;
        cluster_sync_all();
        const int total = nrep * D, per = (total + splits - 1) / splits;
        const int i1 = min(total, (split + 1) * per);
        for (int i = split * per + threadIdx.x; i < i1; i += DEC_THREADS) {
            const int h = i / D, j = i - h * D;
            float mv[8], av[8], lv[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const bool in = u < splits;
                mv[u] = in ? ld_dsmem(cl + nrep * D + h, (uint32_t)u) : -INFINITY;
                av[u] = in ? ld_dsmem(cl + i, (uint32_t)u) : 0.f;
                lv[u] = in ? ld_dsmem(cl + nrep * D + nrep + h, (uint32_t)u) : 0.f;
            }
            float big = -INFINITY;
#pragma unroll
            for (int u = 0; u < 8; ++u) big = fmaxf(big, mv[u]);
            float a = 0.f, lsum = 0.f;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const float wgt = mv[u] == -INFINITY ? 0.f : expf(mv[u] - big);
                a += av[u] * wgt;
                lsum += lv[u] * wgt;
            }
            out[((size_t)row * nh + kvh * nrep + h) * D + j] = from_f<bf16>(a / lsum);
        }
        cluster_sync_all();        // nobody leaves while its shared memory may still be read
        return;
    }
    if (splits > 1 && tickets != nullptr) {
        // The CTA that takes the last ticket of its (request, kv head) merges the splits, in split
        // order; nobody waits for anybody.  The counter is zero again when the launch ends.
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) s_last = atomicAdd(&tickets[bi * nkv + kvh], 1) == splits - 1;
        __syncthreads();
        if (s_last) {
            __threadfence();
            for (int i = threadIdx.x; i < nrep * D; i += DEC_THREADS) {
                const int h = i / D, j = i - h * D;
                const int head = kvh * nrep + h;
                const float* pr = partial + ((size_t)bi * nh + head) * splits * (D + 2);
                // Pieces of 8 splits: all loads of a piece are issued before any is used (one trip
                // to L2 a piece), and the pieces are folded with the running maximum.  With up to
                // 8 splits this is the plain merge: big = max m, sums of acc and l times exp(m - big).
                constexpr int MU = 8;
                float big = -INFINITY, a = 0.f, lsum = 0.f;
                for (int sp0 = 0; sp0 < splits; sp0 += MU) {
                    float mv[MU], av[MU], lv[MU];
#pragma unroll
                    for (int u = 0; u < MU; ++u) {
                        const bool in = sp0 + u < splits;
                        const float* r = pr + (size_t)(in ? sp0 + u : 0) * (D + 2);
                        mv[u] = in ? __ldcg(r + D) : -INFINITY;
                        av[u] = in ? __ldcg(r + j) : 0.f;
                        lv[u] = in ? __ldcg(r + D + 1) : 0.f;
                    }
                    float nb = big;
#pragma unroll
                    for (int u = 0; u < MU; ++u) nb = fmaxf(nb, mv[u]);
                    if (nb == -INFINITY) continue;              // no split of this piece held a key
                    const float keep = big == -INFINITY ? 0.f : expf(big - nb);
                    a *= keep;
                    lsum *= keep;
#pragma unroll
                    for (int u = 0; u < MU; ++u) {              // in the order of the splits
                        const float wgt = mv[u] == -INFINITY ? 0.f : expf(mv[u] - nb);
                        a += av[u] * wgt;
                        lsum += lv[u] * wgt;
                    }
                    big = nb;
                }
                out[((size_t)row * nh + head) * D + j] = from_f<bf16>(a / lsum);
            }
            if (threadIdx.x == 0) tickets[bi * nkv + kvh] = 0;
        }
    }
}

// Ticket counters of the fused merge, part of the library image, zero between launches.  One array
// for every launch of the process that merges by tickets: launches that overlap on the GPU (different
// streams, no dependency between them) would share cells, so callers order them.
constexpr int kMaxTickets = 65536;
__device__ int g_decode_tickets[kMaxTickets];

int g_decode_tma = 1;        // 0: 16-byte asynchronous copies for every size (measurements)
int g_decode_cluster = 1;    // 0: merge through global memory and tickets even where a cluster could (measurements)
int g_decode_stages = 0;     // 0: chosen from the grid; 2..4 for measurements (rlis_attention_decode_set_stages)
int g_decode_last_variant = 0;   // of the last launch: bit 0 tensor-core kernel, bit 1 keys by TMA, bit 2 cluster merge

template <int D, int NSTAGE, bool TMA> constexpr size_t decode_mma_smem_bytes() {
    return (size_t)DEC_WARPS * NSTAGE * 2 * 32 * (TMA ? D : D + 8) * sizeof(bf16);
}

// Merges the splits: big = max m over non-empty splits, w = exp(m - big),
// out = sum acc * w / sum l * w (crates/model/src/paged_attention.metal:276-304).
__global__ void attn_decode_combine_kernel(const float* __restrict__ partial, bf16* __restrict__ out,
                                           const int* __restrict__ dec_rows, int nh, int d,
                                           int splits) {
    pdl_wait_and_trigger();
    const int bi = blockIdx.y, head = blockIdx.x;
    const float* pr = partial + ((size_t)bi * nh + head) * splits * (d + 2);
    float big = -INFINITY;
    for (int s = 0; s < splits; ++s) big = fmaxf(big, pr[(size_t)s * (d + 2) + d]);
    const int row = dec_rows[bi];
    for (int j = threadIdx.x; j < d; j += blockDim.x) {
        float a = 0.f, lsum = 0.f;
        for (int s = 0; s < splits; ++s) {
            const float* r = pr + (size_t)s * (d + 2);
            const float w = r[d] == -INFINITY ? 0.f : expf(r[d] - big);
            a += r[j] * w;
            lsum += r[d + 1] * w;
        }
        out[((size_t)row * nh + head) * d + j] = from_f<bf16>(a / lsum);
    }
}

size_t decode_smem_bytes(int nrep, int d) {
    const int groups = 32 / (d / 8);
    return sizeof(float) * ((size_t)nrep * d + DEC_WARPS * 32 * nrep + (size_t)DEC_WARPS * groups * nrep * d +
                            (size_t)DEC_WARPS * nrep * 2);
}

}  // namespace

// Floats of scratch that `rlis_attention_decode` needs for these sizes (0 when splits == 1).
// Which kernel the last launch of this file took (for tests): bit 0 the tensor-core kernel, bit 1
// keys by bulk tensor copies, bit 2 pieces merged in a cluster, bits 4.. stages of keys.
extern "C" int rlis_attention_decode_last_variant(void) { return g_decode_last_variant; }
extern "C" void rlis_attention_decode_set_stages(int stages) { g_decode_stages = stages; }
extern "C" void rlis_attention_decode_set_cluster(int on) { g_decode_cluster = on; }
extern "C" void rlis_attention_decode_set_tma(int on) { g_decode_tma = on; }
extern "C" int rlis_attention_decode_error(void) { return tc::read_error_word(); }
extern "C" int* rlis_attention_decode_error_addr(void) { return tc::error_word_addr(); }


extern "C" long long rlis_attention_decode_scratch_floats(int n_decode, int nh, int d, int splits) {
    return splits > 1 ? (long long)n_decode * nh * splits * (d + 2) : 0;
}

namespace {
int decode_launch(const void* q, const void* k_cache, const void* v_cache, void* out, float* partial,
                  const int* dec_rows, const int* dec_seqs, const int* ctx_lens, const int* block_tables,
                  int max_blocks, int n_decode, int nh, int nkv, int d, int page_size, float scale,
                  int window, int splits, int dtype, cudaStream_t stream, const DecodeQkv& fz, int n_pages) {
    if (n_decode <= 0) return 0;
    if (dtype != RLIS_BF16 || d % 8 != 0 || d > 256 || d < 8 || nkv <= 0 || nh % nkv != 0 || splits < 1)
        return RLIS_ERR_UNSUPPORTED;
    const int nrep = nh / nkv;
    if (nrep > 8) return RLIS_ERR_UNSUPPORTED;
    if (splits > 1 && partial == nullptr) return RLIS_ERR_UNSUPPORTED;
    if (fz.qkv != nullptr && d != 64 && d != 128) return RLIS_ERR_UNSUPPORTED;   // only the tensor-core kernel rotates
    dim3 grid(nkv, n_decode, splits);
    const size_t smem = decode_smem_bytes(nrep, d);
    bool launched = false;
    bool merged = false;
    if (d == 64 || d == 128) {
        int* tickets = nullptr;
        if (splits > 1 && (long long)n_decode * nkv <= kMaxTickets) {
            static int* ticket_ptr[64] = {nullptr};
            int dev = -1;
            if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64) {
                if (ticket_ptr[dev] == nullptr) {
                    int* p = nullptr;
                    if (cudaGetSymbolAddress((void**)&p, g_decode_tickets) == cudaSuccess) ticket_ptr[dev] = p;
                }
                tickets = ticket_ptr[dev];
            }
        }
        // 2, 4 or 8 splits (8: the portable cluster size) of a grid of a few waves are merged inside
        // a cluster; other sizes schedule badly, and large grids lose more to the clusters' placement
        // than the merge through global memory costs (batch 64: 117 against 110 us)
        int sms = 148, dev = 0;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        const long long ctas = (long long)grid.x * grid.y * grid.z;
        const bool cluster = g_decode_cluster && (splits == 2 || splits == 4 || splits == 8) && ctas <= 4ll * sms;
        merged = tickets != nullptr || cluster;
        // Stages of K/V a warp keeps: what shared memory allows for the CTAs to be resident together
        // (bytes in flight an SM are what the kernel's rate is made of; see the file's head).
        int stages = g_decode_stages;
        // three stages (two CTAs an SM) unless two (three CTAs an SM) get the grid through in
        // fewer rounds (four stages, one CTA an SM, measured slower at every size)
        if (stages == 0) stages = (ctas + 2 * sms - 1) / (2 * sms) <= (ctas + 3 * sms - 1) / (3 * sms) ? 3 : 2;
        if (d == 128 && stages > 3) stages = 3;               // 4 stages of 128-wide rows do not fit
        // Pages of 8 tokens or more (that divide, or are divided by, a block of 32 keys): the keys come
        // by bulk tensor copies into swizzled tiles.  Needs the number of pages (the tensor's bounds);
        // without it, and for other page sizes, 16-byte asynchronous copies.
        const long long cache_rows = (long long)n_pages * nkv * page_size;
        bool tma = g_decode_tma && n_pages > 0 && page_size >= 8 &&
                   (32 % page_size == 0 || page_size % 32 == 0) && cache_rows < (1ll << 31) &&
                   ((reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 15) == 0;
        CUtensorMap map_k = {}, map_v = {};
        if (tma) {
            const int box_rows = page_size < 32 ? page_size : 32;
            tma = tc::make_map(&map_k, k_cache, (int)cache_rows, d, box_rows) &&
                  tc::make_map(&map_v, v_cache, (int)cache_rows, d, box_rows);
        }
#define LAUNCH_MMA(DD, NS, TM)                                                                         \
    do {                                                                                               \
        static bool attr_done = false;                                                                 \
        if (!attr_done) {                                                                              \
            cudaFuncSetAttribute(attn_decode_mma_kernel<DD, NS, TM>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                 (int)decode_mma_smem_bytes<DD, NS, TM>());                            \
            attr_done = true;                                                                          \
        }                                                                                              \
        if (cluster)                                                                                   \
            rlis_launch_cluster(attn_decode_mma_kernel<DD, NS, TM>, grid, DEC_THREADS, decode_mma_smem_bytes<DD, NS, TM>(), \
                stream, dim3(1, 1, (unsigned)splits), map_k, map_v, (int)cache_rows,                   \
                (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out, partial, dec_rows, dec_seqs, \
                ctx_lens, block_tables, max_blocks, nh, nkv, nrep, page_size, scale, window, splits, tickets, fz, 1); \
        else                                                                                           \
            rlis_launch(attn_decode_mma_kernel<DD, NS, TM>, grid, DEC_THREADS, decode_mma_smem_bytes<DD, NS, TM>(), stream, \
                map_k, map_v, (int)cache_rows,                                                         \
                (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out, partial, dec_rows, dec_seqs, \
                ctx_lens, block_tables, max_blocks, nh, nkv, nrep, page_size, scale, window, splits, tickets, fz, 0); \
    } while (0)
        if (d == 64 && tma) {
            if (stages >= 4) LAUNCH_MMA(64, 4, true);
            else if (stages == 3) LAUNCH_MMA(64, 3, true);
            else LAUNCH_MMA(64, 2, true);
        } else if (d == 64) {
            if (stages >= 4) LAUNCH_MMA(64, 4, false);
            else if (stages == 3) LAUNCH_MMA(64, 3, false);
            else LAUNCH_MMA(64, 2, false);
        } else if (tma) {
            if (stages >= 3) LAUNCH_MMA(128, 3, true);
            else LAUNCH_MMA(128, 2, true);
        } else {
            if (stages >= 3) LAUNCH_MMA(128, 3, false);
            else LAUNCH_MMA(128, 2, false);
        }
#undef LAUNCH_MMA
        launched = true;
        g_decode_last_variant = 1 | (tma ? 2 : 0) | (cluster ? 4 : 0) | (stages << 4);
    }
#define LAUNCH(N)                                                                                   \
    rlis_launch(attn_decode_kernel<N>, grid, DEC_THREADS, smem, stream,                                      \
        (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out, partial, dec_rows,  \
        dec_seqs, ctx_lens, block_tables, max_blocks, nh, nkv, d, page_size, scale, window, splits)
    if (!launched) g_decode_last_variant = 0;
    if (!launched) switch (nrep) {
        case 1: LAUNCH(1); break;
        case 2: LAUNCH(2); break;
        case 3: LAUNCH(3); break;
        case 4: LAUNCH(4); break;
        case 5: LAUNCH(5); break;
        case 6: LAUNCH(6); break;
        case 7: LAUNCH(7); break;
        case 8: LAUNCH(8); break;
        default: return RLIS_ERR_UNSUPPORTED;
    }
#undef LAUNCH
    int err = RLIS_LAUNCH_CHECK();
    if (err != 0 || splits == 1 || merged) return err;
    const int threads = d >= 128 ? 128 : (d >= 64 ? 64 : 32);
    rlis_launch(attn_decode_combine_kernel, dim3(nh, n_decode), threads, 0, stream, partial, (bf16*)out, dec_rows, nh, d, splits);
    return RLIS_LAUNCH_CHECK();
}
}  // namespace

extern "C" int rlis_attention_decode(const void* q, const void* k_cache, const void* v_cache,
                                     void* out, float* partial, const int* dec_rows,
                                     const int* dec_seqs, const int* ctx_lens,
                                     const int* block_tables, int max_blocks, int n_decode, int nh,
                                     int nkv, int d, int page_size, float scale, int window,
                                     int splits, int dtype, cudaStream_t stream) {
    const DecodeQkv none = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    return decode_launch(q, k_cache, v_cache, out, partial, dec_rows, dec_seqs, ctx_lens, block_tables, max_blocks,
                         n_decode, nh, nkv, d, page_size, scale, window, splits, dtype, stream, none, 0);
}

// The same with the number of pages of the caches [pages, nkv, page_size, d], which lets the kernel
// fetch keys by bulk tensor copies (see decode_launch).
extern "C" int rlis_attention_decode_pages(const void* q, const void* k_cache, const void* v_cache,
                                           void* out, float* partial, const int* dec_rows,
                                           const int* dec_seqs, const int* ctx_lens,
                                           const int* block_tables, int max_blocks, int n_decode, int nh,
                                           int nkv, int d, int page_size, int n_pages, float scale, int window,
                                           int splits, int dtype, cudaStream_t stream) {
    const DecodeQkv none = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    return decode_launch(q, k_cache, v_cache, out, partial, dec_rows, dec_seqs, ctx_lens, block_tables, max_blocks,
                         n_decode, nh, nkv, d, page_size, scale, window, splits, dtype, stream, none, n_pages);
}

// The same for a step that decodes only, straight from the q|k|v projection [tokens, (nh + 2 nkv) d]
// (head sizes 64 and 128): q and the newest key are rotated inside the kernel (inv_freq == nullptr:
// no rotation) and the newest key and value are stored at slots[token] (slots == nullptr: nothing
// is stored and the cache is taken to hold the key already).  ctx_lens counts the newest key.
extern "C" int rlis_attention_decode_qkv(const void* qkv, const int* positions, const int* slots,
                                         const float* inv_freq, void* k_cache, void* v_cache, void* out,
                                         float* partial, const int* dec_rows, const int* dec_seqs,
                                         const int* ctx_lens, const int* block_tables, int max_blocks,
                                         int n_decode, int nh, int nkv, int d, int page_size, int n_pages,
                                         float scale, int window, int splits, int dtype, cudaStream_t stream) {
    if (qkv == nullptr || positions == nullptr) return RLIS_ERR_UNSUPPORTED;
    const DecodeQkv fz = {(const bf16*)qkv, positions, slots, inv_freq, (bf16*)k_cache, (bf16*)v_cache};
    return decode_launch(nullptr, k_cache, v_cache, out, partial, dec_rows, dec_seqs, ctx_lens, block_tables, max_blocks,
                         n_decode, nh, nkv, d, page_size, scale, window, splits, dtype, stream, fz, n_pages);
}

// ------------------------------------------------------------------------------------------
// The variant that allocates nothing (see attention_decode_static.h for who needs it and the rules).
#include "attention_decode_static.h"

// Part of the library image: every GPU that loads the library holds these 8 MiB until exit.
static __device__ __align__(256) float g_decode_static_scratch[RLIS_DECODE_STATIC_MAX_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
// Device address of the array, per device.  In host code `g_decode_static_scratch` is only a
// stand-in for the symbol, not an address the GPU can use; the address comes from the runtime.
float* g_static_scratch_ptr[kMaxDevices] = {nullptr};
}  // namespace

extern "C" long long rlis_attention_decode_static_capacity(void) { return RLIS_DECODE_STATIC_MAX_FLOATS; }

extern "C" int rlis_attention_decode_static(const void* q, const void* k_cache, const void* v_cache,
                                            void* out, const int* dec_rows, const int* dec_seqs,
                                            const int* ctx_lens, const int* block_tables,
                                            int max_blocks, int n_decode, int nh, int nkv, int d,
                                            int page_size, float scale, int window, int splits,
                                            int dtype, cudaStream_t stream) {
    if (n_decode <= 0) return 0;
    if (rlis_attention_decode_scratch_floats(n_decode, nh, d, splits) > RLIS_DECODE_STATIC_MAX_FLOATS)
        return RLIS_ERR_SCRATCH_TOO_SMALL;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return RLIS_ERR_UNSUPPORTED;
    if (g_static_scratch_ptr[dev] == nullptr) {
        // First call on this device (it is the current one): look the address up once.
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_decode_static_scratch);
        if (e != cudaSuccess) return (int)e;
        g_static_scratch_ptr[dev] = p;
    }
    return rlis_attention_decode(q, k_cache, v_cache, out, g_static_scratch_ptr[dev], dec_rows, dec_seqs,
                                 ctx_lens, block_tables, max_blocks, n_decode, nh, nkv, d, page_size,
                                 scale, window, splits, dtype, stream);
}

// Causal flash attention for portions of prompts over the paged cache on the fifth-generation
// tensor cores (bfloat16, head sizes 64 and 128, two or more query heads per kv head, page
// sizes from 8 on that divide a block of keys: 128 keys for head size 64, 64 for head size 128).  Same contract as attention_prefill.cu (role in the reference: the
// fused `sdpa` call for multi-token segments, crates/model/src/attention.rs:144-157; scores in
// float32, keys after the query hidden, softmax in float32, attention.rs:204-233), which stays
// for the other sizes.
//
// One CTA = 64 tokens of one request x TWO query heads of one kv head: the 128 rows of the tensor
// instruction are (head 0, tokens 0..63), (head 1, tokens 0..63), so every key and value tile is
// used by both heads (a group of three heads is a pair and a head that is taken twice, its copy's
// rows dropped).  Per block of 128 keys:
//   warp 0: TMA.  Q once (two 64 x 64 boxes); the block's K and V page by page (a page of one kv
//           head is a [page_size x 64] box of the cache seen as a 2-D tensor; pages past the
//           context are asked for past the end of the tensor and arrive as zeros), a page a lane,
//           into rings of three tiles for the keys and three for the values, 128-byte swizzle.  A
//           key tile is free once its scores are done, a block earlier than its value tile.
//   warp 1: S = Q K^T (tcgen05.mma, M 128, N 128, K 64) into tensor memory; then O += P V (M 128,
//           N 64, K 128; P is the A operand read from tensor memory, V the MN-major B operand,
//           straight from the cache's layout), accumulated in tensor memory, in two bursts: the
//           first half of the keys as soon as the softmax warps have written that half of P.
//   warps 4-7: a thread per row.  It takes its row of S out of tensor memory at once, finds the
//           maximum, writes P = exp2(s - reference) rounded to bf16 back into tensor memory, two
//           keys to a column.  The reference follows the maximum only when that has run ahead by
//           more than 2^8; then, rarely after the first blocks, the warp rescales its rows of O
//           in tensor memory before the next product.
// Two CTAs fit an SM (112 KB of shared memory, 256 columns of tensor memory each: S 128, O 64,
// P 64) and fill each other's gaps between the phases.  The CTA starts with 128 registers a
// thread; warps 0-3 (two of them idle) give theirs up to 40 and the softmax warps take 216.
//
// What the cycle stamps of an instrumented build showed, and what followed from them (8192 tokens,
// a block of one CTA with two on the SM, before: 3660 cycles):
//   * A burst of tensor instructions costs its issuing thread about 300 cycles before the first is
//     through and 50 each after that, whatever their size (a micro-benchmark of M 128, N 64 ... 256
//     says the same), and the products are done almost as soon as the last is issued.  The eight of
//     P V were 900 cycles between the last exponential and the next block's first; in two bursts
//     the second is 500.
//   * With P in a swizzled tile of shared memory the CTA moved 144 KB a block through shared memory
//     (the products' operands, P written and read, the arriving tiles); with P in tensor memory 80.
//   * The special-function unit does four exponentials a cycle and scheduler: 1024 cycles for a
//     warp's 32 rows of 128 keys.  A lone warp reaches one every 12 cycles, two warps of a
//     scheduler together one every 8.4: the two CTAs of an SM are in their exponentials at the
//     same time most of the time (1900 cycles) and the unit idles in between (a third of the time).
//     More registers for the softmax warps, a three-input maximum in four chains (520 -> 300
//     cycles) and two float32 to an instruction for the scaling and the sums are small change
//     beside that.
//   Now: a block 3040 cycles; 8192 tokens 535 -> 469 us (586 TFLOP/s), 2048 tokens 59 -> 48 us.
//   (Measured and dropped: four heads a CTA with two softmax groups over one ring of tiles and one
//   issuing thread, 627 us at 8192, the thread's bursts one after the other being the bound; the
//   same with the two groups taking turns at the exponentials, 672 us; handing the halves of P
//   back one by one after their own bursts instead of waiting for the whole product, 485 us; eight
//   softmax warps, two threads a row that both read the whole row for the maximum and keep a half
//   each, 512 us: both halves of P are then ready at the same moment, the product's two bursts
//   follow the last exponential one after the other, and the wait for them grows from 400 to 900
//   cycles, more than four warps a scheduler win at the special-function unit.)
//   What is left of a block's 3040 cycles: the exponentials 1900 (the unit's floor for the two
//   CTAs is 2048 a block of both), and the chain last exponential -> P handed over -> second burst
//   (four instructions, their commit 200 cycles, done 170 later) -> the next block's first
//   exponential, about 1000 cycles of which the next block's maximum hides 600.  P cannot be kept
//   twice to take the chain out of the loop: S, O and P fill the CTA's 256 columns.  (Head size 128
//   has the room, S 64 + P 2 x 32 + O 128, and it was measured: 733 -> 723 us at 8192 tokens, 58.4
//   -> 57.2 at 2048; not kept.)
//
// Head size 128 is the same kernel with blocks of 64 keys, so that the tiles are as large and two
// CTAs still fit: a row of Q, K or V is two 128-byte lines, kept as two swizzled sub-tiles of 64
// columns (the scores' eight k-steps take four from each; for P V the value tile is the MN-major
// operand 128 wide, its second sub-tile one leading-dimension offset away), S takes 64 columns of
// tensor memory and O 128, and a thread's row of scores is 64 long.  Per key the tensor work doubles
// and the exponentials do not, so the softmax weighs half as much.  (Head size 64 with blocks of
// 64 keys, 64 KB of tiles, 128 columns of tensor memory and three CTAs an SM was measured too: 60.0
// against 56.9 us at 2048 tokens, 623 against 535 us at 8192: a block's chain of handshakes does
// not shrink with the block.)
//
// (Earlier measurements at 8192 tokens, 32:8 heads, pages of 16: the mma.sync kernel 1356 us.  One
// lane issuing a block's sixteen page copies: 972 us whatever the softmax warps did.  Eight softmax
// warps, two threads a row with a softmax stream and an accumulator each, P in shared memory: 822
// against 706 us.)
//
// A short portion of a long prompt is few tiles with many blocks each: 2 or 4 CTAs of a cluster then
// take a tile's blocks in turn and rank 0 merges their rows through distributed shared memory
// (a 256-token portion at 8192 tokens of context: 114 -> 54 us; with enough tiles to fill the SMs
// the sharing only costs, so it is used when the CTAs fit the SMs at once).
//
// (A whole prompt of 2048 tokens is 512 CTAs for 296 places, and its last tiles are chains of 16
// blocks where a place gets 15 on average.  Sharing only the tiles with more than 11 blocks between
// two CTAs was measured both ways and lost both times: as clusters of two whose second CTA leaves at
// once for a short tile, 56 -> 84 us (a grid of clusters that oversubscribes the SMs schedules
// badly), and as two ordinary CTAs that leave their rows in a scratch buffer for the one that takes
// the tile's last ticket, 57 -> 78 us; at 4096 tokens and more nothing is shared and nothing changes.)
//
// Every mbarrier wait is bounded (a fifth of a second); a wait that runs out sets the error word
// (rlis_attention_prefill_tc_error), every role runs to its end without further waits, and the
// CTA frees its tensor memory before it returns.
#include "tcgen05_utils.cuh"
#include <math.h>

namespace {
using namespace tc;
constexpr int TQ = 64;                  // tokens of a CTA
static_assert(TQ == RLIS_PREFILL_TILE, "the host's tile list is cut for another tile size");
constexpr int TM = 128;                 // rows of the instruction: two heads x 64 tokens
constexpr int MAX_KV_STAGES = 3;
constexpr int PT_THREADS = 256;         // warps 0-3: copies, products and two idle ones; warps 4-7: softmax
constexpr int PT_SOFTMAX_WARP0 = 4;
constexpr int LINE_TILE = TM * 128;     // bytes of a swizzled sub-tile of 128 rows: 64 columns, 128-byte lines
constexpr uint32_t TMEM_COLS = 256;     // S: columns 0 .. TN - 1, O: 128 .. 128 + HD - 1, P (bf16 pairs): TN / 2 columns in what is left

// Sizes by head size HD and keys of a block TN (64, 128) or (128, 64): 16 KB of keys and of values a
// block, three blocks in flight for head size 64 and two for 128 (112 and 96 KB a CTA, two CTAs an SM).
template <int HD, int TN> struct PShape {
    static constexpr int Q_BYTES = TM * HD * 2;             // 16 or 32 KB: HD / 64 sub-tiles [128 x 64]
    static constexpr int KV_TILE_BYTES = TN * HD * 2;       // 16 KB each for K and V: HD / 64 sub-tiles [TN x 64]
    static constexpr int KV_LINE_TILE = TN * 128;           // bytes of one such sub-tile
    static constexpr int KV_STAGES = HD == 64 ? 3 : 2;
    // the tiles + the control block; with the kilobyte the system keeps per CTA, two CTAs fit the
    // 228 KB of an SM only if no alignment slack is spent: the dynamic array is declared 1024-aligned
    static constexpr size_t SMEM = Q_BYTES + KV_STAGES * 2 * KV_TILE_BYTES + 256;
    static constexpr uint32_t IDESC_S = idesc_bf16(TM, TN);
    static constexpr uint32_t IDESC_PV = idesc_bf16(TM, HD) | (1u << 16);      // B (V) is MN-major
    static constexpr uint32_t P_COL = HD == 64 ? 192u : 64u;   // where P lives in tensor memory
    static constexpr int ROW_F = HD + 4;                    // floats a row in the clusters' exchange area
    static constexpr int MAX_SPLITS = HD == 64 ? 4 : 2;     // what that area holds: (splits - 1) * 128 rows
    static_assert((MAX_SPLITS - 1) * TM * ROW_F * 4 <= Q_BYTES + KV_STAGES * 2 * KV_TILE_BYTES,
                  "the exchange area of the cluster merge does not fit the tiles");
    static_assert(TN == 64 || TN == 128, "a block of keys");
    static_assert(KV_STAGES <= MAX_KV_STAGES, "the control block's barriers");
    static_assert(TN <= 128 && HD <= 128 && (HD == 64 ? TN / 2 <= 64 : TN + TN / 2 <= 128),
                  "S, P and O share 256 columns of tensor memory");
    static_assert(2 * (SMEM + 1024) <= 228 * 1024, "two CTAs an SM");
};

// Shared-memory descriptor of the MN-major operand V under the 128-byte swizzle: lines of 64 head
// dimensions, 8 keys to a 1024-byte group (the stride field), and, for heads wider than 64, the
// next 64 dimensions `lbo_bytes` further (the leading-dimension field).
__device__ __forceinline__ uint64_t smem_desc_sw128_mn(const void* tile, uint32_t lbo_bytes) {
    const uint64_t addr = (uint64_t)(smem_u32(tile) >> 4) & 0x3FFFull;
    return addr | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

struct PCtrl {
    uint64_t q_full;
    uint64_t k_full[MAX_KV_STAGES], k_empty[MAX_KV_STAGES];     // keys and values have rings of their own: a key
    uint64_t v_full[MAX_KV_STAGES], v_empty[MAX_KV_STAGES];     // tile is free a whole block before its value tile
    uint64_t s_full, s_empty, p_full[2], o_full;    // P arrives in two halves of the block's keys
    uint32_t tmem_base;
    int abort;
};

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <bool MASK>
__device__ __forceinline__ void max_of_chunk(const uint32_t (&v)[32], int c, int kmin, int kmax, float& mx) {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        const int idx = c * 32 + i;
        const float sv = __uint_as_float(v[i]);
        mx = fmaxf(mx, (!MASK || (idx <= kmax && idx >= kmin)) ? sv : -INFINITY);
    }
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ void max_of_chunk3(const uint32_t (&v)[32], float& mx) {
    float m[4] = {mx, -INFINITY, -INFINITY, -INFINITY};      // four chains: one would be 16 dependent instructions
#pragma unroll
    for (int i = 0; i < 32; i += 8)
#pragma unroll
        for (int j = 0; j < 4; ++j) m[j] = max3(m[j], __uint_as_float(v[i + 2 * j]), __uint_as_float(v[i + 2 * j + 1]));
    mx = max3(m[0], m[1], fmaxf(m[2], m[3]));
}

// Two float32 to an instruction (the softmax warps are bound by the instructions they issue as
// much as by the special-function unit): d = a * b + c and acc += a on pairs.
__device__ __forceinline__ uint64_t pair_of(float x) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %1};" : "=l"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ void fma2(float& d0, float& d1, float a0, float a1, uint64_t b, uint64_t c) {
    asm("{\n.reg .b64 ra, rd;\nmov.b64 ra, {%2, %3};\nfma.rn.f32x2 rd, ra, %4, %5;\nmov.b64 {%0, %1}, rd;\n}\n"
        : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "l"(b), "l"(c));
}
__device__ __forceinline__ void add2(uint64_t& acc, uint32_t a0, uint32_t a1) {
    asm("{\n.reg .b64 ra;\nmov.b64 ra, {%1, %2};\nadd.rn.f32x2 %0, %0, ra;\n}\n" : "+l"(acc) : "r"(a0), "r"(a1));
}
__device__ __forceinline__ float sum_of_pair(uint64_t acc) {
    float lo, hi;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(acc));
    return lo + hi;
}

// P = exp2(s * scale - m) of 32 keys, rounded to bf16, into the row's lane of tensor memory: two
// consecutive keys to a column, the layout in which the tensor core reads its A operand from there.
// `lsum2`: the running sums of the even and of the odd keys.
template <bool MASK>
__device__ __forceinline__ void exp_of_chunk(const uint32_t (&v)[32], int c, int kmin, int kmax, uint64_t scale2,
                                             uint64_t neg_m2, uint32_t tmem_p_row, uint64_t& lsum2) {
    uint32_t pk[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int idx = c * 32 + 2 * i;
        float x0, x1;
        fma2(x0, x1, __uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]), scale2, neg_m2);
        float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
        if (MASK) {
            if (!(idx <= kmax && idx >= kmin)) p0 = 0.f;
            if (!(idx + 1 <= kmax && idx + 1 >= kmin)) p1 = 0.f;
        }
        // the sum is of the rounded values, the ones the product with V uses: the rounding of a
        // dominant key then cancels between numerator and denominator
        const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
        pk[i] = *reinterpret_cast<const uint32_t*>(&h);
        add2(lsum2, pk[i] << 16, pk[i] & 0xffff0000u);
    }
    tmem_st16(tmem_p_row + (uint32_t)(c * 16), pk);
}

// 32 float32 sums of a row, times `inv`, as bf16 to `dst` (16-byte stores).
__device__ __forceinline__ void store_chunk(const uint32_t (&v)[32], float inv, bf16* dst) {
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
        uint4 pk;
        pk.x = pack_bf16(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv);
        pk.y = pack_bf16(__uint_as_float(v[i + 2]) * inv, __uint_as_float(v[i + 3]) * inv);
        pk.z = pack_bf16(__uint_as_float(v[i + 4]) * inv, __uint_as_float(v[i + 5]) * inv);
        pk.w = pack_bf16(__uint_as_float(v[i + 6]) * inv, __uint_as_float(v[i + 7]) * inv);
        *reinterpret_cast<uint4*>(dst + i) = pk;
    }
}
// A row of the accumulated output from tensor memory, normalised, to `orow`.
template <int HD>
__device__ __forceinline__ void store_row(uint32_t tmem_row, float inv, bool pred, bf16* orow) {
#pragma unroll 1
    for (int c = 0; c < HD / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_row + (uint32_t)(c * 32), v);
        if (pred) store_chunk(v, inv, orow + c * 32);
    }
}

// A row's softmax reference may lag behind its maximum by this much (in powers of two) before the
// accumulated output is rescaled: P then holds values up to 2^8, which bf16 and the float32 sums
// take, and the rescaling of O in tensor memory becomes rare after the first blocks.
constexpr float RESCALE_AFTER = 8.0f;

template <int HD, int TN>
__global__ __launch_bounds__(PT_THREADS, 2) void attn_prefill_tc_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out, const int* __restrict__ tiles,
    const int* __restrict__ cu_seqlens, const int* __restrict__ ctx_lens,
    const int* __restrict__ block_tables, int max_blocks, int nh, int nkv, int page_size,
    int cache_rows, float scale, int window, int splits) {
    extern __shared__ __align__(1024) unsigned char pt_smem_raw[];
    if ((smem_u32(pt_smem_raw) & 1023u) != 0u) {       // the swizzled tiles need it; never seen, but checked
        if (threadIdx.x == 0) atomicExch(&g_tc_error, 2);
        return;
    }
    using SH = PShape<HD, TN>;
    constexpr int Q_BYTES = SH::Q_BYTES, KV_TILE_BYTES = SH::KV_TILE_BYTES;
    constexpr int KV_LINE_TILE = SH::KV_LINE_TILE, KV_STAGES = SH::KV_STAGES;
    constexpr int HALVES = HD / 64;                                   // sub-tiles of 64 columns in a row of Q, K, V
    unsigned char* q_tile = pt_smem_raw;
    unsigned char* kv_tiles = q_tile + Q_BYTES;                       // [stage][K|V]
    PCtrl* ctrl = reinterpret_cast<PCtrl*>(kv_tiles + KV_STAGES * 2 * KV_TILE_BYTES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nrep = nh / nkv;
    // x: the pair of heads, y: the tile; CTAs start in the order of the tile list across all heads.
    // The query heads of a kv head go in pairs; with an odd number the last pair holds its one head
    // twice, and the copy's rows are not stored.
    const int b = tiles[2 * blockIdx.y], t0 = tiles[2 * blockIdx.y + 1];
    const int pairs = (nrep + 1) / 2;
    const int pidx = blockIdx.x / splits;
    const int kvh = pidx / pairs;
    const int head0 = kvh * nrep + (pidx % pairs) * 2;
    const bool two = (pidx % pairs) * 2 + 1 < nrep;
    const int head1 = two ? head0 + 1 : head0;
    const int rank = blockIdx.x % splits;                    // of this CTA in its cluster: it takes blocks rank, rank + splits, ...
    const int q_start = cu_seqlens[b];
    const int q_len = cu_seqlens[b + 1] - q_start;
    const int ctx = ctx_lens[b];
    const int pos0 = ctx - q_len + t0;                       // position of the tile's first token
    const int n_valid = min(TQ, q_len - t0);
    const int* table = block_tables + (size_t)b * max_blocks;
    const int last_pos = pos0 + n_valid - 1;
    const int blk_lo = window > 0 ? max(0, pos0 - window + 1) / TN : 0;
    const int blk_hi = last_pos / TN;                        // inclusive
    const int n_blk_all = blk_hi - blk_lo + 1;
    const int n_blk = rank < n_blk_all ? (n_blk_all - rank + splits - 1) / splits : 0;
    const int blk0 = blk_lo + rank;

    if (threadIdx.x == 0) {
        ctrl->abort = 0;
        bar_init(&ctrl->q_full, 1);
        for (int s = 0; s < KV_STAGES; ++s) {
            bar_init(&ctrl->k_full[s], 1);
            bar_init(&ctrl->k_empty[s], 1);
            bar_init(&ctrl->v_full[s], 1);
            bar_init(&ctrl->v_empty[s], 1);
        }
        bar_init(&ctrl->s_full, 1);
        bar_init(&ctrl->s_empty, 4);
        bar_init(&ctrl->p_full[0], 4);
        bar_init(&ctrl->p_full[1], 4);
        bar_init(&ctrl->o_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctrl->tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = ctrl->tmem_base;
    const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 128u, tmem_p = tmem_base + SH::P_COL;
    // warps 4-7: warp w reads TMEM lanes 32 (w % 4) .. + 31; a lane is a row of the tile
    const int srow = (warp & 3) * 32 + lane;
    const uint32_t slane_addr = (uint32_t)((warp & 3) * 32) << 16;
    float m_ref = -INFINITY, l_run = 0.f;       // the reference of the row's exponentials so far, and their sum
    bool row_ok = true;
    // The CTA starts with 128 registers a thread.  The first four warps need few and hand theirs to
    // the softmax warps, which hold a row of 128 scores each and want room beside it to keep several
    // exponentials in flight (with 168 registers for everybody a block took 3700 cycles of a lone
    // CTA, with 206 it took 2900).
    pdl_wait();             // q and this portion's keys come from the kernels before

    if (warp < PT_SOFTMAX_WARP0) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
      if (warp == 0) {
        // producer.  A block of keys is 128 / page_size pages for K and as many for V, each a copy
        // of its own: the lanes of the warp issue them side by side (one lane issuing sixteen
        // copies of 2 KB a block was what bounded the kernel).
        if (lane == 0) {
            bar_expect_tx(&ctrl->q_full, Q_BYTES);
#pragma unroll
            for (int hf = 0; hf < HALVES; ++hf) {        // sub-tile hf: rows 0..63 head 0, rows 64..127 head 1
                tma_load_2d(q_tile + hf * LINE_TILE, &map_q, head0 * HD + hf * 64, q_start + t0, &ctrl->q_full);
                tma_load_2d(q_tile + hf * LINE_TILE + LINE_TILE / 2, &map_q, head1 * HD + hf * 64, q_start + t0,
                            &ctrl->q_full);
            }
        }
        const int pages_per_blk = TN / page_size;
        const int page_bytes = page_size * 128;          // of a page's lines in one sub-tile
        // one tile (the keys or the values of block `it`): a page a lane
        auto load_tile = [&](int it, bool is_v) {
            const int s = it % KV_STAGES;
            uint64_t* full = is_v ? &ctrl->v_full[s] : &ctrl->k_full[s];
            if (it >= KV_STAGES &&
                !bar_wait(is_v ? &ctrl->v_empty[s] : &ctrl->k_empty[s], ((it / KV_STAGES) - 1) & 1, &ctrl->abort))
                return false;
            unsigned char* tile = kv_tiles + (size_t)s * 2 * KV_TILE_BYTES + (is_v ? KV_TILE_BYTES : 0);
            if (lane == 0) bar_expect_tx(full, KV_TILE_BYTES);
            __syncwarp();
            if (lane < pages_per_blk * HALVES) {
                const int pg = lane % pages_per_blk, hf = lane / pages_per_blk;
                const int key = (blk0 + it * splits) * TN + pg * page_size;
                // a page past the context, or wholly behind the window of the tile's first token
                // (it may have been given back): a coordinate past the end of the tensor, zeros arrive
                const bool wanted = key < ctx && (window <= 0 || key + page_size > pos0 - window + 1);
                const int row = wanted ? (table[key / page_size] * nkv + kvh) * page_size : cache_rows;
                tma_load_2d(tile + (size_t)hf * KV_LINE_TILE + (size_t)pg * page_bytes, is_v ? &map_v : &map_k, hf * 64, row, full);
            }
            __syncwarp();
            return true;
        };
        // in the order they are wanted: the keys of a block are multiplied while the block before
        // is in its softmax, its values only after its own
        for (int it = 0; it <= n_blk; ++it) {
            if (it < n_blk && !load_tile(it, false)) break;
            if (it >= 1 && !load_tile(it - 1, true)) break;
        }
      } else if (warp == 1) {
        // The whole warp walks the loop and waits; one lane issues.  (With the loop inside
        // `if (lane == 0)` a product's eight instructions took 800 cycles to issue and every wait on
        // a barrier that was long complete 250: the block's chain P ready -> P V done was 1200
        // cycles for 256 of tensor work.)
        {
            bool ok = bar_wait(&ctrl->q_full, 0, &ctrl->abort);
            uint64_t qdesc[HALVES];
#pragma unroll
            for (int hf = 0; hf < HALVES; ++hf) qdesc[hf] = smem_desc_sw128(q_tile + hf * LINE_TILE);
            auto issue_s = [&](int it) {
                const int s = it % KV_STAGES;
                if (!bar_wait(&ctrl->k_full[s], (it / KV_STAGES) & 1, &ctrl->abort)) return false;
                // the softmax warps have taken the scores of the block before out of tensor memory
                if (it > 0 && !bar_wait(&ctrl->s_empty, (it - 1) & 1, &ctrl->abort)) return false;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned char* kt = kv_tiles + (size_t)s * 2 * KV_TILE_BYTES;
                if (lane == 0) {
#pragma unroll
                    for (int k = 0; k < HD / 16; ++k) {
                        // four k-steps of 32 bytes inside a sub-tile of 64 columns, then the next sub-tile
                        const uint64_t kdesc = smem_desc_sw128(kt + (size_t)(k / 4) * KV_LINE_TILE);
                        umma_bf16(tmem_s, qdesc[k / 4] + (uint64_t)((k % 4) * 32 >> 4), kdesc + (uint64_t)((k % 4) * 32 >> 4),
                                  SH::IDESC_S, k != 0 ? 1u : 0u);
                    }
                    umma_commit(&ctrl->s_full);
                    umma_commit(&ctrl->k_empty[s]);
                }
                __syncwarp();
                return true;
            };
            if (ok && n_blk > 0) ok = issue_s(0);
            for (int it = 0; it < n_blk && ok; ++it) {
                const int s = it % KV_STAGES;
                if (it + 1 < n_blk && !issue_s(it + 1)) break;         // the next block's scores, behind this block's softmax
                // the values have been there for a while; P is what the product waits for
                if (!bar_wait(&ctrl->v_full[s], (it / KV_STAGES) & 1, &ctrl->abort)) break;
                const unsigned char* vt = kv_tiles + (size_t)s * 2 * KV_TILE_BYTES + KV_TILE_BYTES;
                // O += P V in two bursts: the first half of the keys while the softmax warps are in the
                // exponentials of the second (a burst costs 300 cycles before its first instruction
                // is through and 50 an instruction; after the last exponential only four are left)
                bool fine = true;
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    if (!bar_wait(&ctrl->p_full[hf], it & 1, &ctrl->abort)) { fine = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    if (lane == 0) {
#pragma unroll
                        for (int k = hf * (TN / 32); k < (hf + 1) * (TN / 32); ++k) {
                            // P: 16 keys are 8 columns of tensor memory; V: 16 keys = 2 KB further in each of
                            // its sub-tiles of 64 head dimensions
                            const uint64_t vdesc = HALVES == 1 ? smem_desc_sw128(vt + (size_t)k * 16 * 128)
                                                               : smem_desc_sw128_mn(vt + (size_t)k * 16 * 128, (uint32_t)KV_LINE_TILE);
                            umma_bf16_ts(tmem_o, tmem_p + (uint32_t)(k * 8), vdesc, SH::IDESC_PV, (it | k) != 0 ? 1u : 0u);   // O accumulates over the blocks
                        }
                        if (hf == 1) {
                            umma_commit(&ctrl->o_full);
                            umma_commit(&ctrl->v_empty[s]);
                        }
                    }
                    __syncwarp();
                }
                if (!fine) break;
                __syncwarp();
            }
        }
      }
      if (splits > 1) {         // the two meetings of the cluster around the exchange of rows (below)
          __syncwarp();
          cluster_sync_all();
          __syncwarp();
          cluster_sync_all();
      }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
        // softmax and output
        const int r = srow;
        const int pos = pos0 + (srow & 63);
        const int lo = window > 0 ? max(0, pos - window + 1) : 0;
        const uint32_t lane_addr = slane_addr;
        const float scale_log2 = scale * 1.4426950408889634f;
        const uint32_t tmem_p_row = tmem_p + lane_addr;
        bool ok = true;
        for (int it = 0; it < n_blk; ++it) {
            const int key0 = (blk0 + it * splits) * TN;
            ok = bar_wait(&ctrl->s_full, it & 1, &ctrl->abort) && ok;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // the whole row of scores at once, and tensor memory is free for the next block's scores
            uint32_t s0[32], s1[32], s2[TN > 64 ? 32 : 1], s3[TN > 64 ? 32 : 1];
            tmem_ld32_nowait(tmem_s + lane_addr, s0);
            tmem_ld32_nowait(tmem_s + lane_addr + 32u, s1);
            if constexpr (TN > 64) {
                tmem_ld32_nowait(tmem_s + lane_addr + 64u, s2);
                tmem_ld32_nowait(tmem_s + lane_addr + 96u, s3);
            }
            tmem_ld_wait();
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) bar_arrive(&ctrl->s_empty);
            // masks are needed on the causal edge (and with a window) only
            const bool need_mask = key0 + TN - 1 > pos0 || window > 0;
            const int kmax = pos - key0, kmin = lo - key0;           // visible: kmin <= index <= kmax
            float mx = -INFINITY;
            if (need_mask) {
                max_of_chunk<true>(s0, 0, kmin, kmax, mx);
                max_of_chunk<true>(s1, 1, kmin, kmax, mx);
                if constexpr (TN > 64) {
                    max_of_chunk<true>(s2, 2, kmin, kmax, mx);
                    max_of_chunk<true>(s3, 3, kmin, kmax, mx);
                }
            } else {
                max_of_chunk3(s0, mx);
                max_of_chunk3(s1, mx);
                if constexpr (TN > 64) {
                    max_of_chunk3(s2, mx);
                    max_of_chunk3(s3, mx);
                }
            }
            const float m_new = fmaxf(m_ref, mx * scale_log2);
            // the reference moves only when the maximum has run ahead of it (always on the first keys seen)
            const bool move = m_new - m_ref > RESCALE_AFTER || (m_ref == -INFINITY && m_new != -INFINITY);
            float corr = 1.0f;
            if (move) {
                corr = ex2_approx(m_ref - m_new);                    // 0 when nothing was seen before
                m_ref = m_new;
                l_run *= corr;
            }
            const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
            // the product P V of the block before: P may be overwritten and O rescaled once it is done
            // (handing the halves of P back one by one, each after its own part of the product, was
            // measured: the waits it adds cost more than the wait it saves, 485 against 469 us at 8192)
            if (it > 0) {
                ok = bar_wait(&ctrl->o_full, (it - 1) & 1, &ctrl->abort) && ok;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (__any_sync(0xffffffffu, move)) {
#pragma unroll 1
                    for (int c = 0; c < HD / 32; ++c) {
                        uint32_t v[32];
                        tmem_ld32(tmem_o + lane_addr + (uint32_t)(c * 32), v);
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * corr);
                        tmem_st32(tmem_o + lane_addr + (uint32_t)(c * 32), v);
                    }
                    tmem_st_wait();
                }
            }
            // Slots of the last page past the context hold whatever was there before; a zero of P
            // times a NaN would still be a NaN, so those rows of V are cleared (thread r: key r of
            // the block), once the tile has arrived and before any of P is handed over
            if (key0 + TN > ctx) {
                ok = bar_wait(&ctrl->v_full[it % KV_STAGES], (it / KV_STAGES) & 1, &ctrl->abort) && ok;
                if (r < TN && key0 + r >= ctx) {
#pragma unroll
                    for (int hf = 0; hf < HALVES; ++hf) {
                        uint4* vrow = reinterpret_cast<uint4*>(kv_tiles + (size_t)(it % KV_STAGES) * 2 * KV_TILE_BYTES + KV_TILE_BYTES +
                                                               (size_t)hf * KV_LINE_TILE + (size_t)r * 128);
#pragma unroll
                        for (int i = 0; i < 8; ++i) vrow[i] = make_uint4(0u, 0u, 0u, 0u);
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // for the tensor core's reads of V
            }
            // P goes to tensor memory in two halves of the block's keys, each handed to the product
            // as soon as it is complete (O, if it was rescaled, is back there before the first)
            const uint64_t scale2 = pair_of(scale_log2), neg_m2 = pair_of(-m_use);
            uint64_t lsum2 = 0ull;
            auto hand_over = [&](int half) {
                tmem_st_wait();
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) bar_arrive(&ctrl->p_full[half]);
            };
            if (need_mask) {
                exp_of_chunk<true>(s0, 0, kmin, kmax, scale2, neg_m2, tmem_p_row, lsum2);
                if constexpr (TN == 64) hand_over(0);
                exp_of_chunk<true>(s1, 1, kmin, kmax, scale2, neg_m2, tmem_p_row, lsum2);
                if constexpr (TN > 64) {
                    hand_over(0);
                    exp_of_chunk<true>(s2, 2, kmin, kmax, scale2, neg_m2, tmem_p_row, lsum2);
                    exp_of_chunk<true>(s3, 3, kmin, kmax, scale2, neg_m2, tmem_p_row, lsum2);
                }
            } else {
                exp_of_chunk<false>(s0, 0, kmin, kmax, scale2, neg_m2, tmem_p_row, lsum2);
                if constexpr (TN == 64) hand_over(0);
                exp_of_chunk<false>(s1, 1, kmin, kmax, scale2, neg_m2, tmem_p_row, lsum2);
                if constexpr (TN > 64) {
                    hand_over(0);
                    exp_of_chunk<false>(s2, 2, kmin, kmax, scale2, neg_m2, tmem_p_row, lsum2);
                    exp_of_chunk<false>(s3, 3, kmin, kmax, scale2, neg_m2, tmem_p_row, lsum2);
                }
            }
            l_run += sum_of_pair(lsum2);
            hand_over(1);
        }
        if (n_blk > 0) {
            ok = bar_wait(&ctrl->o_full, (n_blk - 1) & 1, &ctrl->abort) && ok;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        row_ok = ok;
        // the row's place in the output: head (srow / 64) of the pair, token (srow % 64) of the tile
        const bool srow_valid = (srow & 63) < n_valid && (srow < 64 || two);
        bf16* sorow = out + ((size_t)(q_start + t0 + (srow & 63)) * nh + (srow < 64 ? head0 : head1)) * HD;
        if (splits == 1) {
            if (n_blk > 0) store_row<HD>(tmem_o + slane_addr, 1.0f / l_run, row_ok && srow_valid, sorow);
        } else {
            // The CTAs of the cluster took the blocks of keys in turn.  Once all their products are done
            // (the tiles in shared memory are free), ranks 1.. send their rows (64 unnormalised sums,
            // the reference of the exponentials and their sum) into rank 0's tiles; rank 0 brings them
            // to one reference in the order of the ranks, adds, normalises and stores.
            constexpr int ROW_F = SH::ROW_F;               // floats a row in the exchange area (16-byte aligned rows)
            float* xchg = reinterpret_cast<float*>(pt_smem_raw);
            __syncwarp();
            cluster_sync_all();
            if (rank > 0) {
                float* dst = xchg + ((size_t)(rank - 1) * TM + srow) * ROW_F;
                uint32_t raddr;
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(raddr) : "r"(smem_u32(dst)), "r"(0));
    #pragma unroll 1
                for (int c = 0; c < HD / 32; ++c) {
                    uint32_t v[32];
                    if (n_blk > 0) {
                        tmem_ld32(tmem_o + slane_addr + (uint32_t)(c * 32), v);
                    } else {
    #pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = 0u;            // no block of its own: nothing was accumulated
                    }
    #pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(raddr + (uint32_t)((c * 32 + i) * 4)),
                                     "r"(v[i]), "r"(v[i + 1]), "r"(v[i + 2]), "r"(v[i + 3]) : "memory");
                }
                asm volatile("st.shared::cluster.v2.b32 [%0], {%1, %2};" ::"r"(raddr + (uint32_t)(HD * 4)),
                             "r"(__float_as_uint(m_ref)), "r"(__float_as_uint(row_ok ? l_run : __int_as_float(0x7fc00000))) : "memory");
            }
            __syncwarp();
            cluster_sync_all();
            if (rank == 0) {
                float m = m_ref;
                for (int k = 1; k < splits; ++k) m = fmaxf(m, xchg[((size_t)(k - 1) * TM + srow) * ROW_F + HD]);
                const float f0 = m_ref == -INFINITY ? 0.f : ex2_approx(m_ref - m);
                float l = l_run * f0;
                float fk[3] = {0.f, 0.f, 0.f};
    #pragma unroll
                for (int k = 1; k < 4; ++k) {
                    if (k < splits) {
                        const float* src = xchg + ((size_t)(k - 1) * TM + srow) * ROW_F;
                        fk[k - 1] = src[HD] == -INFINITY ? 0.f : ex2_approx(src[HD] - m);
                        l += src[HD + 1] * fk[k - 1];
                    }
                }
                const float inv = 1.0f / l;
    #pragma unroll 1
                for (int c = 0; c < HD / 32; ++c) {
                    uint32_t v[32];
                    if (n_blk > 0) {
                        tmem_ld32(tmem_o + slane_addr + (uint32_t)(c * 32), v);
                    } else {
    #pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = 0u;
                    }
    #pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * f0);
    #pragma unroll
                    for (int k = 1; k < 4; ++k) {
                        if (k >= splits) continue;
                        const float4* src = reinterpret_cast<const float4*>(xchg + ((size_t)(k - 1) * TM + srow) * ROW_F + c * 32);
    #pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float4 o = src[i];
                            v[4 * i] = __float_as_uint(fmaf(o.x, fk[k - 1], __uint_as_float(v[4 * i])));
                            v[4 * i + 1] = __float_as_uint(fmaf(o.y, fk[k - 1], __uint_as_float(v[4 * i + 1])));
                            v[4 * i + 2] = __float_as_uint(fmaf(o.z, fk[k - 1], __uint_as_float(v[4 * i + 2])));
                            v[4 * i + 3] = __float_as_uint(fmaf(o.w, fk[k - 1], __uint_as_float(v[4 * i + 3])));
                        }
                    }
                    if (row_ok && srow_valid && l == l) store_chunk(v, inv, sorow + c * 32);
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
    pdl_trigger();
}

// A [rows, cols] bf16 row-major matrix as a 2-D tensor map with boxes of 64 columns x box_rows rows.
bool make_map_2d(CUtensorMap* map, const void* ptr, long long rows, long long cols, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int g_pf_splits = 0;      // 0: chosen from the number of tiles and the longest context
}  // namespace

extern "C" int rlis_attention_prefill_tc_error(void) { return tc::read_error_word(); }
extern "C" int* rlis_attention_prefill_tc_error_addr(void) { return tc::error_word_addr(); }

// 0: automatic; 1, 2 or 4: the CTAs that share a tile's keys.  For measurements.
extern "C" void rlis_attention_prefill_tc_set_splits(int splits) { g_pf_splits = splits; }

// Whether the tensor-core kernel takes these sizes (else the caller uses rlis_attention_prefill).
extern "C" int rlis_attention_prefill_tc_takes(int nh, int nkv, int d, int page_size) {
    if ((d != 64 && d != 128) || nkv <= 0 || nh % nkv != 0 || nh / nkv < 2) return 0;
    const int tn = d == 64 ? 128 : 64;                  // keys of a block
    if (page_size < 8 || page_size > tn || tn % page_size != 0) return 0;
    return 1;
}

namespace {
template <int HD, int TN>
int launch_prefill_tc(const CUtensorMap& map_q, const CUtensorMap& map_k, const CUtensorMap& map_v, bf16* out,
                      const int* tiles, int n_tiles, const int* cu_seqlens, const int* ctx_lens, const int* block_tables,
                      int max_blocks, int nh, int nkv, int page_size, int cache_rows, float scale, int window, int max_ctx,
                      cudaStream_t stream) {
    using SH = PShape<HD, TN>;
    const int pairs = nkv * ((nh / nkv + 1) / 2);          // CTAs a tile: the query heads of a kv head in pairs
    static bool attr_done = false;
    if (!attr_done) {
        cudaFuncSetAttribute(attn_prefill_tc_kernel<HD, TN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SH::SMEM);
        attr_done = true;
    }
    // Few tiles with many keys each (a short portion of a long prompt) would leave SMs idle, and the
    // tiles at the end of a prompt run long after the others are done: 2 or 4 CTAs of a cluster then
    // share a tile's blocks of keys.  max_ctx: the longest context of the step (0: unknown, no sharing).
    int splits = g_pf_splits;
    if (splits <= 0) {
        int dev = 0, sms = 148;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        const long long ctas = (long long)n_tiles * pairs;
        const int blocks = window > 0 ? (window + TQ + TN - 1) / TN + 1 : (max_ctx + TN - 1) / TN;
        splits = 1;
        // measured: it pays while the CTAs still fit the SMs at once (two each) and every one keeps 8 blocks
        while (splits < SH::MAX_SPLITS && ctas * splits * 2 <= 2ll * sms && blocks >= 16 * splits) splits *= 2;
    }
    if (splits > SH::MAX_SPLITS) splits = SH::MAX_SPLITS;
    if (splits != 1 && splits != 2 && splits != 4) return RLIS_ERR_UNSUPPORTED;
    rlis_launch_cluster(attn_prefill_tc_kernel<HD, TN>, dim3((unsigned)(pairs * splits), (unsigned)n_tiles), PT_THREADS,
                        SH::SMEM, stream, dim3((unsigned)splits, 1, 1), map_q, map_k, map_v, out, tiles, cu_seqlens,
                        ctx_lens, block_tables, max_blocks, nh, nkv, page_size, cache_rows, scale, window, splits);
    return RLIS_LAUNCH_CHECK();
}
}  // namespace

// q, out [tokens, nh * d]; caches [pages, nkv, page_size, d]; tiles [n_tiles, 2] = (batch entry,
// first token of 64) as for rlis_attention_prefill; max_ctx: the longest context among the
// requests of the step, or 0.
extern "C" int rlis_attention_prefill_tc(const void* q, const void* k_cache, const void* v_cache, void* out,
                                         const int* tiles, int n_tiles, const int* cu_seqlens,
                                         const int* ctx_lens, const int* block_tables, int max_blocks,
                                         int n_tokens, int n_pages, int nh, int nkv, int d, int page_size,
                                         float scale, int window, int dtype, int max_ctx, cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (dtype != RLIS_BF16 || !rlis_attention_prefill_tc_takes(nh, nkv, d, page_size) || n_tiles > 65535)
        return RLIS_ERR_UNSUPPORTED;
    if (((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) |
          reinterpret_cast<uintptr_t>(out)) & 15) != 0)
        return RLIS_ERR_UNSUPPORTED;
    const long long cache_rows = (long long)n_pages * nkv * page_size;
    if (cache_rows >= (1ll << 31)) return RLIS_ERR_UNSUPPORTED;
    CUtensorMap map_q, map_k, map_v;
    if (!make_map_2d(&map_q, q, n_tokens, (long long)nh * d, TQ) ||
        !make_map_2d(&map_k, k_cache, cache_rows, d, page_size) ||
        !make_map_2d(&map_v, v_cache, cache_rows, d, page_size))
        return RLIS_ERR_UNSUPPORTED;
    if (d == 64)
        return launch_prefill_tc<64, 128>(map_q, map_k, map_v, (bf16*)out, tiles, n_tiles, cu_seqlens, ctx_lens, block_tables,
                                          max_blocks, nh, nkv, page_size, (int)cache_rows, scale, window, max_ctx, stream);
    return launch_prefill_tc<128, 64>(map_q, map_k, map_v, (bf16*)out, tiles, n_tiles, cu_seqlens, ctx_lens, block_tables,
                                      max_blocks, nh, nkv, page_size, (int)cache_rows, scale, window, max_ctx, stream);
}

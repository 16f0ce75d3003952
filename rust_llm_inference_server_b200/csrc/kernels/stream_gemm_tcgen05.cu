// Weight-streaming matrix product for the decode step on the fifth-generation tensor cores:
//   y[M, N] = x[M, K] W[N, K]^T,  bf16 operands, float32 accumulation, M (tokens) up to 128.
// Role of the reference's small-batch GEMV (crates/model/src/gemv.metal:24-94: every weight block
// read once for all rows of the batch).  With a handful of rows the product is a pure stream of W
// from HBM, so the kernel is built to keep bytes in flight with almost no instructions:
//
//   * the weights are the M side of the tensor instruction: a CTA owns 128 output features and a
//     range of k; a 128 x 64 tile of W (16 KB) arrives by ONE bulk tensor copy (TMA, 128-byte
//     swizzle) into a ring of 4 stages, together with the NT x 64 tile of x (NT = tokens rounded
//     up to 16, 32, 64 or 128; rows past M are zero-filled by TMA);
//   * one thread issues tcgen05.mma (M 128, N NT, K 16) into a 128 x NT float32 accumulator in
//     tensor memory; tcgen05.commit frees the stage;
//   * four warps read the accumulator (a lane = a feature, a column = a token) and store.
// Matrices with few features would fill few SMs, so k is split over the CTAs of a thread-block
// cluster (grid = feature tiles x splits, up to 16 splits, about two CTAs an SM and all resident at
// once: the whole matrix is requested in the first microsecond).  After a cluster barrier (all
// products done, the stages free) each CTA sends its float32 partial sums of token t into the
// shared memory of CTA t % splits (st.async, counted on that CTA's mbarrier), which adds the rows
// it was sent in the order of the splits: the result does not depend on timing, nothing passes
// through global memory, and no CTA waits for another one at the end.  The number of splits depends on N and K only, never on the rows, so a token's
// result does not depend on its neighbours.
//
// With more than 16 rows that exchange is slow: every counted store is an update of the finisher's
// one mbarrier, and a tile of 64 rows spent 5 of its 13 us sending (timestamps in the kernel).
// Tiles of 32 and 64 rows are summed by features instead: the 128 features of a tile are 16 chunks
// of 8, chunk c is finished by CTA c % splits, and a thread sends the sums of its feature for 16
// tokens as four plain 16-byte stores into a [sender][4 tokens][feature][token] area of the
// finisher (the 8 lanes of a chunk write 128 contiguous bytes); a second cluster barrier makes them
// visible, and the finisher's threads add the senders in split order for (feature, token) pairs and
// store 8 features of a token side by side.  The order of the additions is the same as before, so
// the result is too.
//
// The first stages of W are requested before the kernel waits for its predecessor in the stream
// (programmatic dependent launch): weights are written by nobody, so the stream of weights goes
// on across the kernel boundary, and only x and y wait.
//
// (Measured on the four products of a 1B Llama layer, 8 rows, 121.6 MB of weights, replayed back
// to back from a graph: an mma.sync kernel fed by 16-byte cp.async copies into per-lane slots,
// 8 features a CTA with its warps splitting k, took 42.0 us a layer, bound by instruction issue
// (about 60 instructions per 512 bytes) and by re-reading x in every CTA; variants of it with bulk
// copies and an mbarrier ring, with whole tiles per warp, or persistent with register double
// buffering were slower still.  This kernel takes 38.4 us without and 34.4 us with the early
// weight requests; the LM head, 525 MB, takes 80 us, the time of a plain copy.  Summing the
// splits through global memory with a ticket per tile instead of the cluster cost 5 us a product.
// Sending a row of partial sums as one bulk copy from a staging area in shared memory, counted once
// on the finisher's mbarrier, instead of 128 counted stores, with the cluster barrier at the end
// that the staging area then needs: 5.6 -> 6.6 us for the QKV product of 8 rows, the step 0.87 ->
// 0.93 ms.  With 17 to 32 rows a layer's four products take 39 us, with 64 rows 51 us (46 and 64 us
// while those tiles were summed token by token), against 39 us for the library (plus its gating
// kernel), and in the step the library is as fast at 32 rows and faster with larger matrices, so
// batches of more than 16 rows go to the library GEMM.)
//
// Epilogues: bf16 or float32 y, or SwiGLU on a gate|up matrix whose rows are interleaved in blocks
// of 4 (rows 8t..8t+3 gate, 8t+4..8t+7 up): y[m, 4t + j] = silu(gate_j) * up_j.
//
// The RMSNorm between two products of a decode step costs a kernel of its own although it moves a
// few kilobytes.  Two more epilogues take it apart and into the products on either side (the
// product is linear in x, so the norm's scale of a row may be applied after it):
//   * "sink" (the last product of a mixer or feed-forward): the finisher adds its result, rounded
//     to bf16 as the unfused path rounds it, to the float32 residual stream in place, writes
//     xn = bf16(resid * norm_weight) for the product that follows, and the sum of resid^2 over
//     its 128 features of every token into partials[tile][token] (a fixed tree over the CTA);
//   * "scaled rows" (the first product of the next part): x is such an xn; the finisher multiplies
//     its sums by 1 / sqrt(sum of the token's partials in the order of the tiles / dim + eps).
// Both are deterministic and depend on the token's own values only.
//
// Every mbarrier wait is bounded (a fifth of a second); a wait that runs out sets an error word
// (rlis_stream_gemm_error), every role runs to its end without further waits, and the CTA frees
// its tensor memory before it returns.
#include "tcgen05_utils.cuh"
#include <math.h>

namespace {
using namespace tc;
constexpr int SF = 128;                 // features of a CTA (the M side of the instruction)
constexpr int SK = 64;                  // k of a stage: 128 bytes of bf16, one swizzle row
constexpr int S_STAGES = 4;             // with x tiles of 16 rows; see stages_of
// Stages of the ring by the rows of the x tile.  Three CTAs have to fit an SM (the clusters of two
// kernels are resident at the same time): with four stages and x tiles of 32 rows only two did,
// and a product of 17 to 32 rows took twice as long as one of 16 (a layer's four products:
// 76 us; with three stages 46 us, with two 54 us).  The stages also hold the rows that the
// cluster sends for the reduction, up to NT + 15 of them (checked in the kernel): two stages of
// 128-row tiles are too small for that.
template <int NT> __host__ __device__ constexpr int stages_of() { return NT <= 16 ? S_STAGES : 3; }
constexpr int W_STAGE_BYTES = SF * SK * 2;
constexpr int S_THREADS = 128;
constexpr int MAX_SPLITS = 16;          // the largest cluster (above 8 is opt-in)

template <int NT> constexpr size_t stream_smem_bytes(int n_stages = stages_of<NT>()) {
    return (size_t)n_stages * (W_STAGE_BYTES + NT * SK * 2) + 1024 /* alignment */ + 768 /* SCtrl */;
}

// A timeline for measurements, compiled in only with -DRLIS_TIMELINE (the build adds it when the
// environment has RLIS_TIMELINE=1; even switched off it cost the decode step 1 %): the first CTA of
// every launch stamps the global timer at its phases into a ring of records, which the host reads
// after a step.  With it a step replayed from a graph can be laid out product by product without a
// tracing tool.
//   0 start, 1 the wait for the kernel before has passed, 2 the products are done, 3 the cluster's
//   barrier, 4 the partial sums are sent, 5 the sums for this CTA's tokens have arrived, 7 end;
//   6 holds N * 100000 + K; 8 the latest end of any CTA of the streaming product launched before
//   (read after the wait: when that whole grid was done, not only its first CTA).
constexpr int TL_RECORDS = 512;
#ifdef RLIS_TIMELINE
__device__ int g_timeline_on;
__device__ unsigned int g_timeline_n;
__device__ unsigned long long g_timeline[TL_RECORDS][10];
__device__ unsigned long long g_timeline_last_end;
#define TL_STAMP(i) do { if (tl_on) g_timeline[tl_slot][i] = now_ns(); } while (0)
#else
#define TL_STAMP(i) do { } while (0)
#endif

struct SCtrl {
    uint64_t full[S_STAGES];
    uint64_t empty[S_STAGES];
    uint64_t acc_full;
    uint64_t red_full;      // the partial sums of the tokens this CTA finishes have arrived from the cluster
    uint32_t tmem_base;
    int abort;
    float red[4];           // sink epilogue: the warps' sums of squares
    float rstd[128];        // scaled rows: the norm's scale of every token
};

// What the two norm epilogues need (all null / 0 when unused).
struct NormFuse {
    const float* in_partials;   // [n_partials, M]: sums of squares of the rows x was made from
    int n_partials;
    int dim;                    // the norm's width
    float eps;
    float* resid;               // sink: [M, N] float32, updated in place
    const float* norm_w;        // sink: [N] weight of the norm that follows
    bf16* xn;                   // sink: [M, N] = bf16(resid * norm_w)
    float* out_partials;        // sink: [tiles, M]
};

// A float into the shared memory of the cluster's CTA `rank` (at the offset of `local`), counted
// on that CTA's mbarrier (at the offset of `bar`).
__device__ __forceinline__ void st_async_f32(float* local, float v, uint64_t* bar, uint32_t rank) {
    uint32_t raddr, rbar;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(raddr) : "r"(smem_u32(local)), "r"(rank));
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rbar) : "r"(smem_u32(bar)), "r"(rank));
    asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];"
                 ::"r"(raddr), "r"(__float_as_uint(v)), "r"(rbar) : "memory");
}

// Four floats into the shared memory of the cluster's CTA `rank` (16-byte aligned), a plain store:
// a cluster barrier orders it before the reads.
__device__ __forceinline__ void st_cluster_f32x4(float* local, uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t rank) {
    uint32_t raddr;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(raddr) : "r"(smem_u32(local)), "r"(rank));
    asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(raddr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// Tiles of 32 and 64 rows are summed by chunks of 8 features (see the head of the file).
template <int NT> __host__ __device__ constexpr bool by_features() { return NT == 32 || NT == 64; }
constexpr int CHUNK_F = 8;                   // features of a chunk
constexpr int N_CHUNKS = SF / CHUNK_F;       // 16 chunks a tile

template <int EPI, typename OutT>
__device__ __forceinline__ void store_token(OutT* __restrict__ y, float v, int t, int f, int lane, int N) {
    if (EPI == 1) {
        // lanes 8i..8i+3 hold gate, 8i+4..8i+7 the matching up values
        const float other = __shfl_xor_sync(0xffffffffu, v, 4);
        if ((lane & 4) == 0 && f + 4 < N)
            y[(size_t)t * (N >> 1) + ((f >> 3) << 2) + (f & 3)] = from_f<OutT>(v / (1.0f + expf(-v)) * other);
    } else if (f < N) {
        y[(size_t)t * N + f] = from_f<OutT>(v);
    }
}

// Sink epilogue for token t, called by all threads of the CTA together (it holds two barriers):
// the thread's feature f of resid += bf16(v); xn = bf16(resid * w); the CTA's sum of resid^2 to
// partials[tile][t].  `live` false: the barriers only.
__device__ __forceinline__ void sink_token(const NormFuse& nf, float* red, float v, int t, int f, int tile, int M,
                                           int N, bool live, float r_old, float w) {
    float r = 0.f;
    if (live && f < N) {
        r = r_old + __bfloat162float(__float2bfloat16_rn(v));
        nf.resid[(size_t)t * N + f] = r;
        nf.xn[(size_t)t * N + f] = __float2bfloat16_rn(r * w);
    }
    const float s = warp_sum(r * r);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0 && live) nf.out_partials[(size_t)tile * M + t] = (red[0] + red[1]) + (red[2] + red[3]);
    __syncthreads();
}

template <int NT, int EPI, typename OutT>
__global__ __launch_bounds__(S_THREADS) void stream_gemm_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                const __grid_constant__ CUtensorMap map_x,
                                                                OutT* __restrict__ y, int M, int N, int K,
                                                                int kb_per_split, int n_stages, const NormFuse nf) {
    extern __shared__ unsigned char sg_smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(sg_smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int X_STAGE_BYTES = NT * SK * 2;
    constexpr uint32_t TMEM_COLS = NT < 32 ? 32 : NT;
    constexpr uint32_t IDESC = idesc_bf16(SF, NT);
    unsigned char* w_tiles = base;
    constexpr int STG = stages_of<NT>();
    static_assert(by_features<NT>() || (size_t)(NT + MAX_SPLITS - 1) * SF * 4 <= (size_t)STG * (W_STAGE_BYTES + NT * SK * 2),
                  "the stages must hold the rows of partial sums that the cluster sends");
    // by features: up to N_CHUNKS + splits - 1 (chunk, sender) blocks of 8 features x NT floats
    static_assert(!by_features<NT>() || (size_t)(N_CHUNKS + MAX_SPLITS - 1) * CHUNK_F * NT * 4 <= (size_t)STG * (W_STAGE_BYTES + NT * SK * 2),
                  "the stages must hold the blocks of partial sums that the cluster sends");
    // A CTA with fewer blocks of k than the ring has stages never wraps around and is given only the
    // stages it uses (n_stages, the same for the whole launch): a product with little k per CTA then
    // takes half the shared memory and fits beside the kernels before and after it, whose CTAs it
    // would otherwise have to wait for before it can request its weights.
    unsigned char* x_tiles = base + (size_t)n_stages * W_STAGE_BYTES;
    SCtrl* ctrl = reinterpret_cast<SCtrl*>(x_tiles + (size_t)n_stages * X_STAGE_BYTES);

#ifdef RLIS_TIMELINE
    const bool tl_on = blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 64 && g_timeline_on != 0;
    unsigned tl_slot = 0;
    if (tl_on) {
        tl_slot = atomicAdd(&g_timeline_n, 1u) % (unsigned)TL_RECORDS;
        g_timeline[tl_slot][6] = (unsigned long long)N * 100000ull + (unsigned long long)K;
    }
#endif
    TL_STAMP(0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x, split = blockIdx.y, splits = gridDim.y;
    const int n0 = tile * SF;
    const int k_blocks = (K + SK - 1) / SK;
    const int kb0 = split * kb_per_split;
    const int kb1 = min(kb0 + kb_per_split, k_blocks);
    const bool has_work = kb0 < kb1;                        // a split past the end of k adds zeros

    if (threadIdx.x == 0) {
        ctrl->abort = 0;
        for (int s = 0; s < STG; ++s) {
            bar_init(&ctrl->full[s], 1);
            bar_init(&ctrl->empty[s], 1);
        }
        bar_init(&ctrl->acc_full, 1);
        bar_init(&ctrl->red_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // tokens split, split + splits, ... are finished by this CTA: every CTA of the cluster
        // sends a row of 128 floats for each of them
        const int owned = split < M ? (M - split + splits - 1) / splits : 0;
        if (!by_features<NT>() && splits > 1 && owned > 0) bar_expect_tx(&ctrl->red_full, (uint32_t)(owned * splits * SF * 4));
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    }
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctrl->tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = ctrl->tmem_base;

    if (warp == 0 && lane == 0) {
        // producer: one bulk tensor copy per 16 KB of W.  No kernel writes the weights, so the first
        // stages of W are requested before this grid's dependency on the previous kernel of the
        // stream is resolved (programmatic dependent launch); x and y wait for it.
        const int n_kb = kb1 - kb0;
        const int early = n_kb < STG ? n_kb : STG;
        for (int it = 0; it < early; ++it) {
            bar_expect_tx(&ctrl->full[it], W_STAGE_BYTES + X_STAGE_BYTES);
            tma_load_2d(w_tiles + (size_t)it * W_STAGE_BYTES, &map_w, (kb0 + it) * SK, n0, &ctrl->full[it]);
        }
        pdl_wait();
        for (int it = 0; it < early; ++it)
            tma_load_2d(x_tiles + (size_t)it * X_STAGE_BYTES, &map_x, (kb0 + it) * SK, 0, &ctrl->full[it]);
        for (int it = early; it < n_kb; ++it) {
            const int s = it % STG, kb = kb0 + it;
            if (!bar_wait(&ctrl->empty[s], ((it / STG) - 1) & 1, &ctrl->abort)) break;
            bar_expect_tx(&ctrl->full[s], W_STAGE_BYTES + X_STAGE_BYTES);
            tma_load_2d(w_tiles + (size_t)s * W_STAGE_BYTES, &map_w, kb * SK, n0, &ctrl->full[s]);
            tma_load_2d(x_tiles + (size_t)s * X_STAGE_BYTES, &map_x, kb * SK, 0, &ctrl->full[s]);
        }
        pdl_trigger();     // everything this CTA reads is requested: the next kernel may start its own requests
    } else if (warp == 1 && lane == 0) {
        for (int kb = kb0, it = 0; kb < kb1; ++kb, ++it) {
            const int s = it % STG;
            if (!bar_wait(&ctrl->full[s], (it / STG) & 1, &ctrl->abort)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t adesc = smem_desc_sw128(w_tiles + (size_t)s * W_STAGE_BYTES);
            const uint64_t bdesc = smem_desc_sw128(x_tiles + (size_t)s * X_STAGE_BYTES);
#pragma unroll
            for (int k = 0; k < SK / 16; ++k)          // 32 bytes further along K in the swizzled row
                umma_bf16(tmem_base, adesc + (uint64_t)(k * 32 >> 4), bdesc + (uint64_t)(k * 32 >> 4), IDESC,
                          (it | k) != 0 ? 1u : 0u);
            umma_commit(&ctrl->empty[s]);
        }
        if (has_work) umma_commit(&ctrl->acc_full);
    }
    __syncwarp();
    pdl_wait();            // nothing is stored before the kernels before this one have finished
    TL_STAMP(1);
#ifdef RLIS_TIMELINE
    if (tl_on) g_timeline[tl_slot][8] = *reinterpret_cast<volatile unsigned long long*>(&g_timeline_last_end);
#endif
    const bool scaled = EPI != 2 && nf.in_partials != nullptr;
    if (scaled && (int)threadIdx.x < M) {
        // this token's scale: the partial sums in the order of the tiles (RMSNorm: 1 / sqrt(mean + eps))
        float ss = 0.f;
        for (int p = 0; p < nf.n_partials; ++p) ss += nf.in_partials[(size_t)p * M + threadIdx.x];
        ctrl->rstd[threadIdx.x] = 1.0f / sqrtf(ss / (float)nf.dim + nf.eps);
    }
    // sink: what the first token this thread finishes needs from memory, requested before the sums arrive
    const int f = n0 + warp * 32 + lane;
    float sink_w = 0.f, sink_r0 = 0.f;
    if (EPI == 2 && f < N) {
        sink_w = nf.norm_w[f];
        const int t0 = splits == 1 ? 0 : split;
        if (t0 < M) sink_r0 = nf.resid[(size_t)t0 * N + f];
    }
    const bool waited = has_work ? bar_wait(&ctrl->acc_full, 0, &ctrl->abort) : true;
    const bool ok = __syncthreads_and(waited ? 1 : 0) != 0;       // the same for all threads
    TL_STAMP(2);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    // epilogue: warp w reads TMEM lanes 32 w .. 32 w + 31; lane = feature, column = token
    const uint32_t tmem_acc = tmem_base + ((uint32_t)(warp * 32) << 16);
    if (splits == 1) {
#pragma unroll 1
        for (int c = 0; c < NT / 16; ++c) {
            if (c * 16 >= M) break;
            uint32_t r[16];
            tmem_ld16(tmem_acc + (uint32_t)(c * 16), r);
            if (EPI == 2) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int t = c * 16 + j;
                    if (t >= M) continue;           // the same for all threads
                    const float r_old = t == 0 ? sink_r0 : (ok && f < N ? nf.resid[(size_t)t * N + f] : 0.f);
                    sink_token(nf, ctrl->red, __uint_as_float(r[j]), t, f, tile, M, N, ok, r_old, sink_w);
                }
                continue;
            }
            if (!ok) continue;
#pragma unroll
            for (int j = 0; j < 16; ++j)
                if (c * 16 + j < M)
                    store_token<EPI, OutT>(y, __uint_as_float(r[j]) * (scaled ? ctrl->rstd[c * 16 + j] : 1.0f),
                                           c * 16 + j, f, lane, N);
        }
    } else {
        // Once every CTA of the cluster is done with its products, the stages are free everywhere:
        // each CTA sends its partial sums of token t to the CTA that finishes t (rank t % splits),
        // into that CTA's stages as [t / splits][sender][feature], counted on its mbarrier.  The
        // finisher waits for its bytes only, adds the rows in the order of the splits, and nobody
        // reads anybody's shared memory, so nobody has to be waited for at the end.
        float* part = reinterpret_cast<float*>(w_tiles);
        cluster_sync_all();
        TL_STAMP(3);
        if constexpr (by_features<NT>()) {
            // this thread's feature belongs to chunk ch, which CTA ch % splits finishes; there it is block
            // (ch / splits) * splits + split, laid out [group of 4 tokens][feature of 8][token of 4]
            const int ch = (int)threadIdx.x / CHUNK_F, fi = (int)threadIdx.x % CHUNK_F;
            float* dst = part + ((ch / splits) * splits + split) * (CHUNK_F * NT) + fi * 4;
            const uint32_t to = (uint32_t)(ch % splits);
#pragma unroll 1
            for (int c = 0; c < NT / 16; ++c) {
                if (c * 16 >= M) break;
                uint32_t r[16];
                if (has_work) {
                    tmem_ld16(tmem_acc + (uint32_t)(c * 16), r);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) r[j] = 0u;
                }
#pragma unroll
                for (int j = 0; j < 16; j += 4)
                    st_cluster_f32x4(dst + ((c * 16 + j) / 4) * (CHUNK_F * 4), r[j], r[j + 1], r[j + 2], r[j + 3], to);
            }
            TL_STAMP(4);
            cluster_sync_all();                 // what was sent has arrived; nobody touches another CTA's memory from here on
            TL_STAMP(5);
            // thread -> feature fi of the chunk and tokens tg, tg + 16, ...: the 8 features of a token are
            // neighbouring lanes (the SwiGLU pairs four lanes apart, 16-byte runs of y)
            const int tg = (int)threadIdx.x / CHUNK_F;
#pragma unroll 1
            for (int c2 = split, slot = 0; c2 < N_CHUNKS; c2 += splits, ++slot) {
                const int fo = n0 + c2 * CHUNK_F + fi;
#pragma unroll 1
                for (int t = tg; t < ((M + 15) & ~15); t += S_THREADS / CHUNK_F) {
                    const float* src = part + (slot * splits) * (CHUNK_F * NT) + (t / 4) * (CHUNK_F * 4) + fi * 4 + (t & 3);
                    float v = 0.f;
                    for (int sdr = 0; sdr < splits; ++sdr) v += src[sdr * (CHUNK_F * NT)];
                    const float sc = scaled && t < M ? ctrl->rstd[t] : 1.0f;
                    if (EPI == 1) {
                        // (every lane takes part in the exchange of the gated epilogue; rows past M are not stored)
                        const float g = v * sc;
                        const float other = __shfl_xor_sync(0xffffffffu, g, 4);
                        if (ok && t < M && (fi & 4) == 0 && fo + 4 < N)
                            y[(size_t)t * (N >> 1) + ((fo >> 3) << 2) + (fo & 3)] = from_f<OutT>(g / (1.0f + expf(-g)) * other);
                    } else if (ok && t < M && fo < N) {
                        y[(size_t)t * N + fo] = from_f<OutT>(v * sc);
                    }
                }
            }
        } else {
#pragma unroll 1
        for (int c = 0; c < NT / 16; ++c) {
            if (c * 16 >= M) break;
            uint32_t r[16];
            if (has_work) {
                tmem_ld16(tmem_acc + (uint32_t)(c * 16), r);
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) r[j] = 0u;
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const int t = c * 16 + j;
                if (t < M)
                    st_async_f32(part + ((t / splits) * splits + split) * SF + (int)threadIdx.x, __uint_as_float(r[j]),
                                 &ctrl->red_full, (uint32_t)(t % splits));
            }
        }
        TL_STAMP(4);
        if (split < M) {
            const bool got = bar_wait(&ctrl->red_full, 0, &ctrl->abort);
            TL_STAMP(5);
            const bool good = EPI == 2 ? __syncthreads_and(ok && got ? 1 : 0) != 0 : (ok && got);
#pragma unroll 1
            for (int t = split, slot = 0; t < M; t += splits, ++slot) {
                float v = 0.f;
                for (int s = 0; s < splits; ++s) v += part[(slot * splits + s) * SF + (int)threadIdx.x];
                if (EPI == 2) {
                    const float r_old = slot == 0 ? sink_r0 : (good && f < N ? nf.resid[(size_t)t * N + f] : 0.f);
                    sink_token(nf, ctrl->red, v, t, f, tile, M, N, good, r_old, sink_w);
                } else if (good) {
                    store_token<EPI, OutT>(y, v * (scaled ? ctrl->rstd[t] : 1.0f), t, f, lane, N);
                }
            }
        }
        }
    }
    TL_STAMP(7);
#ifdef RLIS_TIMELINE
    if (threadIdx.x == 64 && g_timeline_on != 0) atomicMax(&g_timeline_last_end, now_ns());
#endif
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 2) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

int g_target_ctas = 0;      // 0: twice the number of SMs
int g_min_stages = -1;      // stages a CTA is given at least (measurements; -1: by the rows, see launch_stream)

template <int NT, int EPI, typename OutT>
int launch_stream(const void* x, const void* W, void* y, int M, int N, int K, const NormFuse& nf, cudaStream_t stream) {
    CUtensorMap map_w, map_x;
    if (!make_map(&map_w, W, N, K, SF) || !make_map(&map_x, x, M, K, NT)) return RLIS_ERR_UNSUPPORTED;
    static bool attr_done = false;
    if (!attr_done) {
        cudaFuncSetAttribute(stream_gemm_kernel<NT, EPI, OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)stream_smem_bytes<NT>());
        cudaFuncSetAttribute(stream_gemm_kernel<NT, EPI, OutT>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        attr_done = true;
    }
    const int tiles = (N + SF - 1) / SF, k_blocks = (K + SK - 1) / SK;
    int target = g_target_ctas;
    if (target <= 0) {
        int dev = 0, sms = 148;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        target = 2 * sms;
    }
    // splits (the cluster's size, any number up to 16) from N and K alone: about two CTAs an SM, at
    // least two stages of k each, and no split without work.  (Measured in the decode step of a 1B
    // Llama, batch 8: gate|up, 128 tiles, in 3 splits instead of 2: -29 us a step, in 4: +46 us;
    // the O projection, 16 tiles and 32 blocks of k, in 16 instead of 8: -15 us.)
    int splits = (target + tiles - 1) / tiles;
    if (splits > MAX_SPLITS) splits = MAX_SPLITS;
    if (splits > k_blocks / 2) splits = k_blocks / 2;
    if (splits < 1) splits = 1;
    const int per = (k_blocks + splits - 1) / splits;
    splits = (k_blocks + per - 1) / per;
    // stages: what a CTA's blocks of k use, and what the cluster's exchange of partial sums needs
    constexpr int STG = stages_of<NT>();
    const size_t stage_bytes = (size_t)W_STAGE_BYTES + (size_t)NT * SK * 2;
    size_t exchange = 0;
    if (splits > 1)
        exchange = by_features<NT>() ? (size_t)((N_CHUNKS + splits - 1) / splits) * splits * CHUNK_F * NT * 4
                                     : (size_t)((M + splits - 1) / splits) * splits * SF * 4;
    // (Measured in the decode step of a 1B Llama, context 4096.  One request: every product with the
    // stages it uses 0.706 ms, with three at least 0.716, with all four 0.718: the products that fit
    // beside their neighbours request their weights earlier.  Eight requests: 0.883, 0.876 and
    // 0.884 ms: there the kernel before the O projection streams keys and values, and two-stage CTAs
    // of the projection, all resident at once, compete with it.)
    int min_stages = g_min_stages >= 0 ? g_min_stages : (M <= 2 ? 0 : 3);
    int n_stages = per < STG ? per : STG;
    if (n_stages < min_stages) n_stages = min_stages < STG ? min_stages : STG;
    while (n_stages < STG && (size_t)n_stages * stage_bytes < exchange) ++n_stages;
    rlis_launch_cluster(stream_gemm_kernel<NT, EPI, OutT>, dim3((unsigned)tiles, (unsigned)splits), S_THREADS,
                        stream_smem_bytes<NT>(n_stages), stream, dim3(1, (unsigned)splits, 1), map_w, map_x, (OutT*)y, M, N, K,
                        per, n_stages, nf);
    return RLIS_LAUNCH_CHECK();
}

template <int NT>
int dispatch_stream(const void* x, const void* W, void* y, int M, int N, int K, int out_dtype, int epilogue,
                    const NormFuse& nf, cudaStream_t stream) {
    if (epilogue == 0 && out_dtype == RLIS_BF16) return launch_stream<NT, 0, bf16>(x, W, y, M, N, K, nf, stream);
    if (epilogue == 0 && out_dtype == RLIS_F32) return launch_stream<NT, 0, float>(x, W, y, M, N, K, nf, stream);
    if (epilogue == 1 && out_dtype == RLIS_BF16) return launch_stream<NT, 1, bf16>(x, W, y, M, N, K, nf, stream);
    return RLIS_ERR_UNSUPPORTED;
}
}  // namespace

// The timeline of the launches (see g_timeline): switch, and read-out of the ring [512][10] with the
// number of records written so far.  Both synchronise the device.
// Both synchronise the device; RLIS_ERR_UNSUPPORTED from a library built without the timeline.
extern "C" int rlis_stream_gemm_timeline(int on) {
#ifdef RLIS_TIMELINE
    const unsigned int zero = 0;
    cudaError_t e = cudaMemcpyToSymbol(g_timeline_n, &zero, sizeof(zero));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_timeline_on, &on, sizeof(on));
    return (int)e;
#else
    (void)on;
    return RLIS_ERR_UNSUPPORTED;
#endif
}
extern "C" int rlis_stream_gemm_timeline_read(unsigned long long* out, unsigned int* n) {
#ifdef RLIS_TIMELINE
    cudaError_t e = cudaMemcpyFromSymbol(n, g_timeline_n, sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaMemcpyFromSymbol(out, g_timeline, sizeof(unsigned long long) * TL_RECORDS * 10);
    return (int)e;
#else
    (void)out;
    (void)n;
    return RLIS_ERR_UNSUPPORTED;
#endif
}
extern "C" int rlis_stream_gemm_error(void) { return tc::read_error_word(); }
extern "C" int* rlis_stream_gemm_error_addr(void) { return tc::error_word_addr(); }

// About how many CTAs a launch is cut into (0: twice the SMs).  For measurements.
extern "C" void rlis_stream_gemm_set_target(int ctas) { g_target_ctas = ctas; }
extern "C" void rlis_stream_gemm_set_min_stages(int n) { g_min_stages = n; }

// out_dtype: RLIS_BF16 or RLIS_F32.  epilogue 0: y [M, N]; 1 (SwiGLU, rows of W interleaved
// gate/up in blocks of 4, N a multiple of 8): y [M, N / 2].  M up to 128; K a multiple of 8;
// x and W 16-byte aligned.
//
// Scaled rows (epilogues 0 and 1; in_partials not null): x is bf16(resid * norm weight) and
// in_partials [n_partials, M] the sums of squares that a sink product left; y is multiplied by
// 1 / sqrt(sum / norm_dim + eps) of its row.
// Sink (epilogue 2, M up to 16; y unused): resid [M, N] float32 += bf16(x W^T) in place,
// xn [M, N] bf16 = resid * norm_w, out_partials [ceil(N / 128), M] = sums of resid^2 by 128 features.
extern "C" int rlis_stream_gemm_fused(const void* x, const void* W, void* y, int M, int N, int K, int out_dtype,
                                      int epilogue, const float* in_partials, int n_partials, int norm_dim, float eps,
                                      float* resid, const float* norm_w, void* xn, float* out_partials,
                                      cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 128 || K <= 0 || (K & 7) != 0) return RLIS_ERR_UNSUPPORTED;
    if (epilogue == 1 && (N & 7) != 0) return RLIS_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(W) & 15) != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0)
        return RLIS_ERR_UNSUPPORTED;
    NormFuse nf{};
    if (in_partials != nullptr) {
        if (epilogue == 2 || n_partials <= 0 || norm_dim <= 0) return RLIS_ERR_UNSUPPORTED;
        nf.in_partials = in_partials;
        nf.n_partials = n_partials;
        nf.dim = norm_dim;
        nf.eps = eps;
    }
    if (epilogue == 2) {
        if (M > 16 || resid == nullptr || norm_w == nullptr || xn == nullptr || out_partials == nullptr)
            return RLIS_ERR_UNSUPPORTED;
        nf.resid = resid;
        nf.norm_w = norm_w;
        nf.xn = reinterpret_cast<bf16*>(xn);
        nf.out_partials = out_partials;
        return launch_stream<16, 2, bf16>(x, W, nullptr, M, N, K, nf, stream);
    }
    if (M <= 16) return dispatch_stream<16>(x, W, y, M, N, K, out_dtype, epilogue, nf, stream);
    if (M <= 32) return dispatch_stream<32>(x, W, y, M, N, K, out_dtype, epilogue, nf, stream);
    if (M <= 64) return dispatch_stream<64>(x, W, y, M, N, K, out_dtype, epilogue, nf, stream);
    return dispatch_stream<128>(x, W, y, M, N, K, out_dtype, epilogue, nf, stream);
}

extern "C" int rlis_stream_gemm_bf16(const void* x, const void* W, void* y, int M, int N, int K,
                                     int out_dtype, int epilogue, cudaStream_t stream) {
    if (epilogue == 2) return RLIS_ERR_UNSUPPORTED;
    return rlis_stream_gemm_fused(x, W, y, M, N, K, out_dtype, epilogue, nullptr, 0, 0, 0.f, nullptr, nullptr, nullptr,
                                  nullptr, stream);
}

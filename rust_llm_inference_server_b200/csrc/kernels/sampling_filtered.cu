// Temperature sampling with top-k and/or top-p (nucleus) filtering on the device, one CTA per row
// of float32 logits, so that such rows no longer send their logits (half a megabyte at 128 k
// vocabulary) to the host.  The reference filters on the host (crates/engine/src/sampler.rs:116-221:
// weights exp((l - max) / T), the k highest logits, the shortest descending prefix whose share of
// the mass reaches top_p, an inverse-CDF draw); the rule is the same here, arranged so that no
// sort is needed and every sum is exact:
//   * weights are fixed-point integers, w = floor(exp((l - max) / T) * 2^40), added with integer
//     atomics, so sums do not depend on the order of addition and a draw is reproducible;
//   * the k-th highest logit, and then the nucleus threshold (the largest value t with
//     mass{l >= t} >= top_p * mass), are found by a radix search over the order-preserving 32-bit
//     image of the floats: four passes of 8 bits, a 256-bin histogram each (counts for top-k,
//     masses for top-p);
//   * the token is drawn from the kept set by inverse CDF in vocabulary order with a 53-bit
//     uniform that the host derives from (seed, position): r = floor(u * kept mass), the first token
//     whose running mass exceeds r.
// Of logits equal to a threshold the lowest token ids are kept, as the reference's ordering has it.
// params[r] = (bits of 1/T, top_k, bits of top_p, low and high word of the 53-bit uniform).
#include "common.cuh"
#include "mma_utils.cuh"
#include <math.h>

namespace {
constexpr int FT = 1024;
typedef unsigned long long u64;

__device__ __forceinline__ uint32_t order_key(float f) {
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ u64 fixed_weight(float logit, float mx, float inv_t) {
    const float w = expf((logit - mx) * inv_t);           // in (0, 1]
    return (u64)(w * 1099511627776.0f);                    // * 2^40
}
__device__ __forceinline__ u64 block_sum_u64(u64 v, u64* scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        u64 s = lane < FT / 32 ? scratch[lane] : 0ull;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) scratch[32] = s;
    }
    __syncthreads();
    const u64 r = scratch[32];
    __syncthreads();
    return r;
}

__device__ __forceinline__ float key_value(uint32_t key) {
    return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}

// Over the row: how many keys exceed `key0`, how many equal it, and the mass of those that exceed it.
__device__ __forceinline__ void key_stats(const float* row, int vocab, uint32_t key0, float mx, float inv_t,
                                          u64* scratch, u64& n_above, u64& n_ties, u64& mass_above) {
    u64 a = 0ull, t = 0ull, m = 0ull;
    for (int v = threadIdx.x; v < vocab; v += FT) {
        const float l = row[v];
        const uint32_t key = order_key(l);
        if (key > key0) { ++a; m += fixed_weight(l, mx, inv_t); }
        else if (key == key0) ++t;
    }
    n_above = block_sum_u64(a, scratch);
    n_ties = block_sum_u64(t, scratch);
    mass_above = block_sum_u64(m, scratch);
}

__global__ __launch_bounds__(FT) void sample_filtered_kernel(const float* __restrict__ logits,
                                                             const uint32_t* __restrict__ params,
                                                             int* __restrict__ out, int vocab,
                                                             long long row_stride) {
    pdl_wait();
    __shared__ u64 hist[256];
    __shared__ u64 scratch[33];
    __shared__ u64 scan_a[FT / 32], scan_b[FT / 32];
    __shared__ float s_max[FT / 32];
    __shared__ uint32_t s_prefix;
    __shared__ u64 s_above;
    __shared__ int s_owner;
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * row_stride;
    const float inv_t = __uint_as_float(params[5 * r]);
    const int top_k = (int)params[5 * r + 1];
    const float top_p = __uint_as_float(params[5 * r + 2]);
    const u64 u53 = (u64)params[5 * r + 3] | ((u64)params[5 * r + 4] << 32);
    const bool use_k = top_k > 0 && top_k < vocab;
    const bool use_p = top_p < 1.0f;

    // the row's maximum
    float mx = -INFINITY;
    for (int v = threadIdx.x; v < vocab; v += FT) mx = fmaxf(mx, row[v]);
    mx = warp_max(mx);
    if ((threadIdx.x & 31) == 0) s_max[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = s_max[0];
    for (int i = 1; i < FT / 32; ++i) mx = fmaxf(mx, s_max[i]);
    __syncthreads();

    // top-k: the k-th highest key by radix search on counts
    uint32_t kth = 0u;
    if (use_k) {
        uint32_t prefix = 0u;
        u64 k_rem = (u64)top_k;
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            for (int i = threadIdx.x; i < 256; i += FT) hist[i] = 0ull;
            __syncthreads();
            for (int v = threadIdx.x; v < vocab; v += FT) {
                const uint32_t key = order_key(row[v]);
                if (pass == 0 || (key >> (shift + 8)) == (prefix >> (shift + 8)))
                    atomicAdd(&hist[(key >> shift) & 255u], 1ull);
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                u64 cum = 0ull;
                int b = 255;
                for (; b > 0; --b) {
                    if (cum + hist[b] >= k_rem) break;
                    cum += hist[b];
                }
                s_prefix = prefix | ((uint32_t)b << shift);
                s_above = cum;
            }
            __syncthreads();
            prefix = s_prefix;
            k_rem -= s_above;
            __syncthreads();
        }
        kth = prefix;
    }
    // Of the logits equal to the k-th one only as many as top_k still has room for are kept, lowest
    // ids first (crates/engine/src/sampler.rs:182-195).
    u64 n_above_k, n_ties_k, mass_above_k;
    key_stats(row, vocab, kth, mx, inv_t, scratch, n_above_k, n_ties_k, mass_above_k);
    const u64 keep_k = use_k ? (u64)top_k - n_above_k : n_ties_k;
    const u64 w_k = fixed_weight(key_value(kth), mx, inv_t);
    const u64 mass = mass_above_k + keep_k * w_k;        // of the top-k set (or of everything)

    // top-p: the largest threshold whose upper mass reaches top_p * mass, by radix search on masses
    uint32_t thr = kth;
    u64 tie_keep = keep_k;
    if (use_p) {
        const u64 target = (u64)((double)top_p * (double)mass);
        uint32_t prefix = 0u;
        u64 above = 0ull;                     // mass of keys above the bins chosen so far
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            for (int i = threadIdx.x; i < 256; i += FT) hist[i] = 0ull;
            __syncthreads();
            for (int v = threadIdx.x; v < vocab; v += FT) {
                const float l = row[v];
                const uint32_t key = order_key(l);
                if (key >= kth && (pass == 0 || (key >> (shift + 8)) == (prefix >> (shift + 8))))
                    atomicAdd(&hist[(key >> shift) & 255u], fixed_weight(l, mx, inv_t));
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                u64 cum = above;
                int b = 255;
                for (; b > 0; --b) {
                    if (cum + hist[b] >= target && hist[b] > 0ull) break;
                    cum += hist[b];
                }
                s_prefix = prefix | ((uint32_t)b << shift);
                s_above = cum;
            }
            __syncthreads();
            prefix = s_prefix;
            above = s_above;
            __syncthreads();
        }
        thr = prefix > kth ? prefix : kth;
        // of the logits equal to the threshold, the lowest ids are kept until the mass is reached
        // (the crossing token included; sampler.rs:200-209)
        u64 n_above, n_ties, mass_above;
        key_stats(row, vocab, thr, mx, inv_t, scratch, n_above, n_ties, mass_above);
        const u64 w_t = fixed_weight(key_value(thr), mx, inv_t);
        u64 need = 1ull;
        if (target > mass_above && w_t > 0ull) need = (target - mass_above + w_t - 1ull) / w_t;
        if (need < 1ull) need = 1ull;
        const u64 room = thr == kth ? keep_k : n_ties;
        tie_keep = need < room ? need : room;
    }

    // inverse CDF over the kept set in vocabulary order: a contiguous piece of the row per thread
    const int per = (vocab + FT - 1) / FT;
    const int v0 = min(threadIdx.x * per, vocab), v1 = min(v0 + per, vocab);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // rank of this piece's first tie among all logits equal to the threshold
    u64 my_ties = 0ull;
    for (int v = v0; v < v1; ++v) my_ties += order_key(row[v]) == thr ? 1ull : 0ull;
    u64 incl_t = my_ties;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const u64 n = __shfl_up_sync(0xffffffffu, incl_t, o);
        if (lane >= o) incl_t += n;
    }
    if (lane == 31) scan_a[warp] = incl_t;
    __syncthreads();
    u64 tie_rank = incl_t - my_ties;
    for (int i = 0; i < warp; ++i) tie_rank += scan_a[i];
    // kept mass of this piece
    u64 mine = 0ull, rank = tie_rank;
    for (int v = v0; v < v1; ++v) {
        const float l = row[v];
        const uint32_t key = order_key(l);
        if (key > thr || (key == thr && rank++ < tie_keep)) mine += fixed_weight(l, mx, inv_t);
    }
    u64 incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const u64 n = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += n;
    }
    if (lane == 31) scan_b[warp] = incl;
    if (threadIdx.x == 0) s_owner = -1;
    __syncthreads();
    u64 warp_base = 0ull, kept = 0ull;
    for (int i = 0; i < FT / 32; ++i) {
        if (i < warp) warp_base += scan_b[i];
        kept += scan_b[i];
    }
    const u64 before = warp_base + incl - mine;
    // r = floor(u * kept), u = u53 / 2^53
    const u64 target_r = __umul64hi(u53 << 11, kept);
    if (mine > 0ull && target_r >= before && target_r < before + mine) s_owner = threadIdx.x;
    __syncthreads();
    if ((int)threadIdx.x == s_owner) {
        u64 cum = before, rk = tie_rank;
        int pick = v1 - 1;
        for (int v = v0; v < v1; ++v) {
            const float l = row[v];
            const uint32_t key = order_key(l);
            if (key > thr || (key == thr && rk++ < tie_keep)) {
                cum += fixed_weight(l, mx, inv_t);
                if (cum > target_r) { pick = v; break; }
            }
        }
        out[r] = pick;
    }
    if (s_owner < 0 && threadIdx.x == 0) out[r] = 0;   // nothing kept (a row of NaNs): id 0, as the greedy path
    pdl_trigger();   // the next kernel of the stream may start its launch
}

int g_filtered_cluster = 1;      // 0: the one-CTA kernel for every vocabulary (tests of that kernel)

// ------------------------------------------------------------------------------------------------
// The same rule with a thread-block cluster per row.  One CTA reading a row of 128 k logits a dozen
// times took 1.9 ms; here the row is read once: a cluster of CC CTAs of 512 threads holds it in
// registers (thread t of CTA c: E consecutive token ids, so that CTA order and thread order are
// vocabulary order), every pass works on registers, histograms and sums of the CTAs meet through
// distributed shared memory, and every CTA draws the same conclusions from the same totals.  Same
// integers, same token as the one-CTA kernel above, which stays for vocabularies too large for it.
constexpr int CT = 512;

__device__ __forceinline__ u64 ld_dsmem_u64(const u64* local, uint32_t rank) {
    uint32_t remote;
    u64 v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
    asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(remote) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t ld_dsmem_u32(const uint32_t* local, uint32_t rank) {
    uint32_t remote, v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(remote) : "memory");
    return v;
}

// The values at one shared-memory offset in all CTAs of the cluster, added in rank order.
__device__ __forceinline__ u64 cluster_total_u64(const u64* local, uint32_t cc) {
    u64 t = 0ull;
    for (uint32_t c = 0; c < cc; ++c) t += ld_dsmem_u64(local, c);
    return t;
}
__device__ __forceinline__ u64 cluster_total_u32(const uint32_t* local, uint32_t cc) {
    u64 t = 0ull;
    for (uint32_t c = 0; c < cc; ++c) t += ld_dsmem_u32(local, c);
    return t;
}

// Three sums over the CTA at once.  `scratch`: 3 x (CT / 32 + 1) values.
__device__ __forceinline__ void cta_sum3_u64(u64& a, u64& b, u64& c, u64 (*scratch)[CT / 32 + 1]) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        a += __shfl_xor_sync(0xffffffffu, a, o);
        b += __shfl_xor_sync(0xffffffffu, b, o);
        c += __shfl_xor_sync(0xffffffffu, c, o);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { scratch[0][warp] = a; scratch[1][warp] = b; scratch[2][warp] = c; }
    __syncthreads();
    if (warp < 3) {
        u64 s = lane < CT / 32 ? scratch[warp][lane] : 0ull;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) scratch[warp][CT / 32] = s;
    }
    __syncthreads();
    a = scratch[0][CT / 32]; b = scratch[1][CT / 32]; c = scratch[2][CT / 32];
    __syncthreads();
}

// The radix step on 256 totals held one a thread (threads 0..255; `mine` is 0 elsewhere): the highest
// bin b whose totals from the top reach `need` (`base` + sum of bins above b + bin b >= need; with
// `nonempty`, bin b itself must hold something), and the sum of the bins above it.  Bin 0 if none.
// A scan by one thread took 4 us a pass.
__device__ __forceinline__ void pick_bin(u64 mine, u64 base, u64 need, bool nonempty, u64* warp_tot, int* best,
                                         u64* above_out, uint32_t* bin_out) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    u64 incl = mine;                                   // sum of this warp's bins at or above this one
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const u64 n = __shfl_down_sync(0xffffffffu, incl, o);
        if (lane + o < 32) incl += n;
    }
    if (tid < 256 && lane == 0) warp_tot[warp] = incl;
    if (tid == 0) *best = 0;
    __syncthreads();
    u64 above = incl - mine;
    if (tid < 256)
        for (int w = warp + 1; w < 8; ++w) above += warp_tot[w];
    if (tid < 256 && base + above + mine >= need && (!nonempty || mine > 0ull)) atomicMax(best, tid);
    __syncthreads();
    if (tid == *best) {
        *above_out = base + above;
        *bin_out = (uint32_t)tid;
    }
    __syncthreads();
}

struct ClusterShared {
    uint32_t hist_c[2][256];     // counts of a radix pass (two buffers: a pass is read by the others while the next is filled)
    u64 hist_w[2][256];          // masses of a radix pass
    u64 xch[16][3];              // a CTA's sums of a phase, read by the whole cluster
    float xmax;
    u64 scratch3[3][CT / 32 + 1];
    u64 scan[CT / 32];
    uint32_t prefix;
    u64 above;
    u64 warp_tot[8];
    int best;
    uint32_t bin;
};

template <int E>
__global__ __launch_bounds__(CT) void sample_filtered_cluster_kernel(const float* __restrict__ logits,
                                                                     const uint32_t* __restrict__ params,
                                                                     int* __restrict__ out, int vocab,
                                                                     long long row_stride) {
    pdl_wait();
    __shared__ ClusterShared sh;
    const uint32_t rank = blockIdx.x, cc = gridDim.x;
    const int r = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* row = logits + (size_t)r * row_stride;
    const float inv_t = __uint_as_float(params[5 * r]);
    const int top_k = (int)params[5 * r + 1];
    const float top_p = __uint_as_float(params[5 * r + 2]);
    const u64 u53 = (u64)params[5 * r + 3] | ((u64)params[5 * r + 4] << 32);
    const bool use_k = top_k > 0 && top_k < vocab;
    const bool use_p = top_p < 1.0f;
    int phase = 0;                                   // which xch slot the next cluster-wide sum uses

    // this thread's E consecutive tokens
    const int v0 = ((int)rank * CT + tid) * E;
    float lg[E];
    uint32_t key[E];
    bool rows16 = ((reinterpret_cast<uintptr_t>(row) & 15) == 0) && v0 + E <= vocab;
    if (rows16) {
#pragma unroll
        for (int i = 0; i < E; i += 4) {
            const float4 x = *reinterpret_cast<const float4*>(row + v0 + i);
            lg[i] = x.x; lg[i + 1] = x.y; lg[i + 2] = x.z; lg[i + 3] = x.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < E; ++i) lg[i] = v0 + i < vocab ? row[v0 + i] : -INFINITY;
    }
    const int n_mine = max(0, min(E, vocab - v0));   // tokens past the vocabulary take part in nothing

    // the row's maximum
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < E; ++i) {
        if (i < n_mine) mx = fmaxf(mx, lg[i]);
        key[i] = order_key(lg[i]);
    }
    mx = warp_max(mx);
    float* fscr = reinterpret_cast<float*>(sh.scratch3[0]);
    if (lane == 0) fscr[warp] = mx;
    __syncthreads();
    if (tid == 0) {
        float m = fscr[0];
        for (int i = 1; i < CT / 32; ++i) m = fmaxf(m, fscr[i]);
        sh.xmax = m;
    }
    cluster_sync_all();
    mx = -INFINITY;
    for (uint32_t c = 0; c < cc; ++c) mx = fmaxf(mx, ld_dsmem(&sh.xmax, c));
    // weights in float32, once; the fixed-point integer is made from them where needed
    float wf[E];
#pragma unroll
    for (int i = 0; i < E; ++i) wf[i] = expf((lg[i] - mx) * inv_t);
    auto fixed = [&](int i) -> u64 { return (u64)(wf[i] * 1099511627776.0f); };

    // sums of three numbers over the whole cluster, the same in every CTA
    auto cluster_sums = [&](u64& a, u64& b, u64& c3) {
        cta_sum3_u64(a, b, c3, sh.scratch3);
        u64* slot = sh.xch[phase & 15];
        ++phase;
        if (tid == 0) { slot[0] = a; slot[1] = b; slot[2] = c3; }
        cluster_sync_all();
        a = cluster_total_u64(slot, cc);
        b = cluster_total_u64(slot + 1, cc);
        c3 = cluster_total_u64(slot + 2, cc);
    };
    // over the row: keys above `key0`, keys equal to it, mass of those above
    auto key_stats = [&](uint32_t key0, u64& n_above, u64& n_ties, u64& mass_above) {
        u64 a = 0ull, t = 0ull, m = 0ull;
#pragma unroll
        for (int i = 0; i < E; ++i) {
            if (i < n_mine) {
                if (key[i] > key0) { ++a; m += fixed(i); }
                else if (key[i] == key0) ++t;
            }
        }
        cluster_sums(a, t, m);
        n_above = a; n_ties = t; mass_above = m;
    };

    int pass_no = 0;
    // the key of the k-th highest logit, by radix search on counts
    auto count_select = [&](u64 k_rem) -> uint32_t {
        uint32_t prefix = 0u;
        for (int pass = 0; pass < 4; ++pass, ++pass_no) {
            const int shift = 24 - 8 * pass;
            uint32_t* hist = sh.hist_c[pass_no & 1];
            for (int i = tid; i < 256; i += CT) hist[i] = 0u;
            __syncthreads();
            // (logits of one row crowd into a few bins: the lanes of a warp that meet in a bin add up
            // among themselves first, and one of them goes to shared memory)
#pragma unroll
            for (int i = 0; i < E; ++i) {
                const bool in = i < n_mine && (pass == 0 || (key[i] >> (shift + 8)) == (prefix >> (shift + 8)));
                if (!__any_sync(0xffffffffu, in)) continue;
                const uint32_t bin = in ? (key[i] >> shift) & 255u : 256u;
                const uint32_t peers = __match_any_sync(0xffffffffu, bin);
                if (in && lane == __ffs(peers) - 1) atomicAdd(&hist[bin], (uint32_t)__popc(peers));
            }
            cluster_sync_all();
            const u64 tot = tid < 256 ? cluster_total_u32(&hist[tid], cc) : 0ull;
            pick_bin(tot, 0ull, k_rem, false, sh.warp_tot, &sh.best, &sh.above, &sh.bin);
            prefix |= sh.bin << shift;
            k_rem -= sh.above;
            __syncthreads();
        }
        return prefix;
    };
    const uint32_t kth = use_k ? count_select((u64)top_k) : 0u;
    u64 n_above_k, n_ties_k, mass_above_k;
    key_stats(kth, n_above_k, n_ties_k, mass_above_k);
    const u64 keep_k = use_k ? (u64)top_k - n_above_k : n_ties_k;
    const u64 w_k = fixed_weight(key_value(kth), mx, inv_t);
    const u64 mass = mass_above_k + keep_k * w_k;

    // top-p: the largest threshold whose upper mass reaches top_p * mass
    uint32_t thr = kth;
    u64 tie_keep = keep_k;
    if (use_p) {
        const u64 target = (u64)((double)top_p * (double)mass);
        // Without a top-k the search over masses would put every token of the row into histograms
        // of 64-bit sums.  Counting is cheaper: if the PRE highest logits already hold the target
        // mass, the nucleus lies among them and only they take part (the result is the same:
        // the threshold depends on the masses above it alone).
        uint32_t lower = kth;
        constexpr int PRE = 1024;
        if (!use_k && vocab > 4 * PRE) {
            const uint32_t kpre = count_select((u64)PRE);
            u64 n_above, n_ties, mass_above;
            key_stats(kpre, n_above, n_ties, mass_above);
            if (mass_above + n_ties * fixed_weight(key_value(kpre), mx, inv_t) >= target) lower = kpre;
        }
        uint32_t prefix = 0u;
        u64 above = 0ull;
        for (int pass = 0; pass < 4; ++pass, ++pass_no) {
            const int shift = 24 - 8 * pass;
            u64* hist = sh.hist_w[pass_no & 1];
            for (int i = tid; i < 256; i += CT) hist[i] = 0ull;
            __syncthreads();
#pragma unroll
            for (int i = 0; i < E; ++i) {
                const u64 w = fixed(i);
                const bool in = i < n_mine && key[i] >= lower && w != 0ull &&
                                (pass == 0 || (key[i] >> (shift + 8)) == (prefix >> (shift + 8)));
                if (!__any_sync(0xffffffffu, in)) continue;
                const uint32_t bin = in ? (key[i] >> shift) & 255u : 256u;
                const uint32_t peers = __match_any_sync(0xffffffffu, bin);
                // the weights (below 2^41) of the lanes that meet in a bin, added in two 32-bit halves
                const uint32_t lo = __reduce_add_sync(peers, (uint32_t)(w & 0xFFFFFFull));
                const uint32_t hi = __reduce_add_sync(peers, (uint32_t)(w >> 24));
                if (in && lane == __ffs(peers) - 1) atomicAdd(&hist[bin], (u64)lo + ((u64)hi << 24));
            }
            cluster_sync_all();
            const u64 tot = tid < 256 ? cluster_total_u64(&hist[tid], cc) : 0ull;
            pick_bin(tot, above, target, true, sh.warp_tot, &sh.best, &sh.above, &sh.bin);
            prefix |= sh.bin << shift;
            above = sh.above;
            __syncthreads();
        }
        thr = prefix > kth ? prefix : kth;
        u64 n_above, n_ties, mass_above;
        key_stats(thr, n_above, n_ties, mass_above);
        const u64 w_t = fixed_weight(key_value(thr), mx, inv_t);
        u64 need = 1ull;
        if (target > mass_above && w_t > 0ull) need = (target - mass_above + w_t - 1ull) / w_t;
        if (need < 1ull) need = 1ull;
        const u64 room = thr == kth ? keep_k : n_ties;
        tie_keep = need < room ? need : room;
    }

    // An exclusive prefix over the vocabulary order (CTA after CTA, thread after thread) of a value
    // per thread; also the cluster's total.
    auto ordered_prefix = [&](u64 mine, u64& total) -> u64 {
        u64 incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const u64 n = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += n;
        }
        if (lane == 31) sh.scan[warp] = incl;
        __syncthreads();
        u64 before = incl - mine, cta_total = 0ull;
        for (int i = 0; i < CT / 32; ++i) {
            if (i < warp) before += sh.scan[i];
            cta_total += sh.scan[i];
        }
        u64* slot = sh.xch[phase & 15];
        ++phase;
        if (tid == 0) slot[0] = cta_total;
        cluster_sync_all();
        total = 0ull;
        for (uint32_t c = 0; c < cc; ++c) {
            const u64 t = ld_dsmem_u64(slot, c);
            if (c < rank) before += t;
            total += t;
        }
        return before;
    };
    // rank of this thread's first tie among all logits equal to the threshold
    u64 my_ties = 0ull;
#pragma unroll
    for (int i = 0; i < E; ++i) my_ties += (i < n_mine && key[i] == thr) ? 1ull : 0ull;
    u64 all_ties;
    const u64 tie_rank = ordered_prefix(my_ties, all_ties);
    // kept mass of this thread's tokens
    u64 mine = 0ull, rk = tie_rank;
#pragma unroll
    for (int i = 0; i < E; ++i)
        if (i < n_mine && (key[i] > thr || (key[i] == thr && rk++ < tie_keep))) mine += fixed(i);
    u64 kept;
    const u64 before = ordered_prefix(mine, kept);
    const u64 target_r = __umul64hi(u53 << 11, kept);          // floor(u * kept), u = u53 / 2^53
    if (mine > 0ull && target_r >= before && target_r < before + mine) {
        u64 cum = before, rk2 = tie_rank;
        int pick = v0 + n_mine - 1;
#pragma unroll
        for (int i = 0; i < E; ++i) {
            if (i < n_mine && (key[i] > thr || (key[i] == thr && rk2++ < tie_keep))) {
                cum += fixed(i);
                if (cum > target_r) { pick = v0 + i; break; }
            }
        }
        out[r] = pick;
    }
    if (kept == 0ull && rank == 0 && tid == 0) out[r] = 0;     // nothing kept (a row of NaNs): id 0, as the greedy path
    cluster_sync_all();          // nobody leaves while its shared memory may still be read
    pdl_trigger();
}

template <int E>
void launch_filtered_cluster(const float* logits, const uint32_t* params, int* out, int rows, int vocab,
                             long long row_stride, int cc, cudaStream_t stream) {
    static bool attr_done = false;
    if (!attr_done) {
        cudaFuncSetAttribute(sample_filtered_cluster_kernel<E>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        attr_done = true;
    }
    rlis_launch_cluster(sample_filtered_cluster_kernel<E>, dim3((unsigned)cc, (unsigned)rows), CT, 0, stream,
                        dim3((unsigned)cc, 1, 1), logits, params, out, vocab, row_stride);
}
}  // namespace

extern "C" int rlis_sample_filtered(const float* logits, const uint32_t* params, int* out, int rows, int vocab,
                                    long long row_stride, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return RLIS_ERR_UNSUPPORTED;
    // a cluster of 8 (16 for the largest) CTAs of 512 threads holds the row in registers, 8 to 32
    // tokens a thread; vocabularies beyond 262,144 go to the one-CTA kernel
    const long long per8 = ((long long)vocab + 8 * CT - 1) / (8 * CT);
    if (g_filtered_cluster && per8 <= 8) launch_filtered_cluster<8>(logits, params, out, rows, vocab, row_stride, 8, stream);
    else if (g_filtered_cluster && per8 <= 16) launch_filtered_cluster<16>(logits, params, out, rows, vocab, row_stride, 8, stream);
    else if (g_filtered_cluster && per8 <= 32) launch_filtered_cluster<32>(logits, params, out, rows, vocab, row_stride, 8, stream);
    else if (g_filtered_cluster && per8 <= 64) launch_filtered_cluster<32>(logits, params, out, rows, vocab, row_stride, 16, stream);
    else rlis_launch(sample_filtered_kernel, rows, FT, 0, stream, logits, params, out, vocab, row_stride);
    return RLIS_LAUNCH_CHECK();
}

extern "C" void rlis_sample_filtered_set_cluster(int on) { g_filtered_cluster = on; }

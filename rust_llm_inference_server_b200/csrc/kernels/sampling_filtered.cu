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
}  // namespace

extern "C" int rlis_sample_filtered(const float* logits, const uint32_t* params, int* out, int rows, int vocab,
                                    long long row_stride, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return RLIS_ERR_UNSUPPORTED;
    rlis_launch(sample_filtered_kernel, rows, FT, 0, stream, logits, params, out, vocab, row_stride);
    return RLIS_LAUNCH_CHECK();
}

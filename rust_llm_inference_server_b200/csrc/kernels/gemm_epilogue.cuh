// What the epilogue warps of the tcgen05 products do with 32 consecutive float32 sums of one row.
#pragma once
#include "common.cuh"
#include "mma_utils.cuh"

namespace tc {

// EPI 0: bf16 y [M, N].  EPI 1: SwiGLU over a gate|up matrix whose rows are interleaved in blocks of
// 4 (columns 8 t .. 8 t + 3 gate, 8 t + 4 .. 8 t + 7 up), y [M, N / 2] bf16.  EPI 2: float32 y [M, N].
// r: the sums of columns col .. col + 31 of row `row`; columns from N on are not stored.
template <int EPI>
__device__ __forceinline__ void store_sums32(const uint32_t (&r)[32], void* __restrict__ y, int row, int col, int N) {
    if (EPI == 0) {
        bf16* o = reinterpret_cast<bf16*>(y) + (size_t)row * N + col;
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            if (col + v * 8 >= N) break;
            uint4 pk;
            pk.x = pack_bf16(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]));
            pk.y = pack_bf16(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
            pk.z = pack_bf16(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
            pk.w = pack_bf16(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
            *reinterpret_cast<uint4*>(o + v * 8) = pk;
        }
    } else if (EPI == 1) {
        bf16* o = reinterpret_cast<bf16*>(y) + (size_t)row * (N >> 1) + (col >> 1);
        float res[16];
#pragma unroll
        for (int tt = 0; tt < 4; ++tt)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float gt = __uint_as_float(r[tt * 8 + j]), up = __uint_as_float(r[tt * 8 + 4 + j]);
                res[tt * 4 + j] = gt / (1.0f + expf(-gt)) * up;
            }
#pragma unroll
        for (int v = 0; v < 2; ++v) {
            if (col + v * 16 >= N) break;
            uint4 pk;
            pk.x = pack_bf16(res[v * 8 + 0], res[v * 8 + 1]);
            pk.y = pack_bf16(res[v * 8 + 2], res[v * 8 + 3]);
            pk.z = pack_bf16(res[v * 8 + 4], res[v * 8 + 5]);
            pk.w = pack_bf16(res[v * 8 + 6], res[v * 8 + 7]);
            *reinterpret_cast<uint4*>(o + v * 8) = pk;
        }
    } else {
        float* o = reinterpret_cast<float*>(y) + (size_t)row * N + col;
#pragma unroll
        for (int v = 0; v < 8; ++v) {
            if (col + v * 4 >= N) break;
            *reinterpret_cast<float4*>(o + v * 4) = make_float4(
                __uint_as_float(r[v * 4]), __uint_as_float(r[v * 4 + 1]), __uint_as_float(r[v * 4 + 2]),
                __uint_as_float(r[v * 4 + 3]));
        }
    }
}

}  // namespace tc

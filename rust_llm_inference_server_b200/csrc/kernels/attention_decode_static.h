// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in akshajnad/rust_llm_inference_server; it is an addition
// of this library.
//
// Who needs it: a host program that gave the whole GPU to an arena of its own at start-up, so a
// later cudaMalloc would fail or eat into memory it has promised elsewhere; a serving loop that
// cannot afford cudaMalloc's implicit synchronisation of the device in the middle of a step; a
// plug-in that runs inside somebody else's process and may not touch that process's allocator
// (torch's included).  `rlis_attention_decode` asks its caller for a scratch buffer when the
// context is split; those callers have nowhere to get one from.
//
// `rlis_attention_decode_static` is the same kernel with the same arguments, minus `partial`: the
// partial results of the splits go to an array that is part of the library image
// (RLIS_DECODE_STATIC_MAX_FLOATS float32 = 8 MiB; every GPU that loads the library holds that
// much until the process exits).  The caller still passes inputs and the output.
//
// Rules of use:
//  * It calls no cudaMalloc, cudaFree or other allocating routine.
//  * n_decode * nh * splits * (d + 2) must not exceed RLIS_DECODE_STATIC_MAX_FLOATS when
//    splits > 1; otherwise the call returns RLIS_ERR_SCRATCH_TOO_SMALL (-2) and launches nothing.
//  * The first call on a device looks the array's device address up (cudaGetSymbolAddress, with
//    that device current) and keeps it.  Make that first call outside any stream capture.
//  * Every call shares the one array and finds the last call's contents in it.  Nothing in it has
//    to start at zero: each (request, head, split) cell that the merge reads is written by this
//    call's first kernel.  Two calls that overlap on the GPU (different streams, no dependency)
//    race on the array: order them.
//  * The same holds between this entry point and the ordinary ones.  Where the splits are merged by
//    "the last ticket folds", every decode-attention launch of the process, whichever entry point
//    made it, counts its tickets in one array of the library image, indexed by (request, kv head).
//    Two such launches that overlap on the GPU would count into each other's cells, and a merge
//    could run early or not at all.  Launches on one stream are ordered by the stream; launches on
//    different streams have to be ordered by the caller (an event), whatever their scratch buffers.
//  * The two look-ups of device addresses (this array's and the ticket array's) are kept in plain
//    per-device variables.  Two host threads that make the first call on a device at the same time
//    both do the look-up and store the same value; nothing else is shared between host threads.
#pragma once

#include <cuda_runtime.h>

#define RLIS_DECODE_STATIC_MAX_FLOATS (2 * 1024 * 1024)
#define RLIS_ERR_SCRATCH_TOO_SMALL (-2)

#ifdef __cplusplus
extern "C" {
#endif

int rlis_attention_decode_static(const void* q, const void* k_cache, const void* v_cache, void* out,
                                 const int* dec_rows, const int* dec_seqs, const int* ctx_lens,
                                 const int* block_tables, int max_blocks, int n_decode, int nh,
                                 int nkv, int d, int page_size, float scale, int window, int splits,
                                 int dtype, cudaStream_t stream);

// Largest scratch, in float32 elements, that the static entry point can serve.
long long rlis_attention_decode_static_capacity(void);

#ifdef __cplusplus
}
#endif

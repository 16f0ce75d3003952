// Process-wide switches of the kernel library and the error word of its bounded waits.
#include "common.cuh"

#include <string.h>

// Programmatic dependent launch (see common.cuh).  On by default: the decode step (batch 8,
// context 4096, replayed from a graph) measured 1.15 ms with it and 1.27 ms without.  What it buys
// is the weight-streaming product's first requests for weights, which go out while the kernel
// before is still running.
int g_rlis_pdl = 1;

extern "C" void rlis_set_pdl(int on) { g_rlis_pdl = on ? 1 : 0; }
extern "C" int rlis_get_pdl(void) { return g_rlis_pdl; }

// ---- one hook for every measurement and test switch ------------------------------------------
// The kernels choose their own launch shapes; these switches exist so that a measurement or a test
// can hold one choice fixed.  Nothing in the engine sets them.
//   pdl              0 / 1     programmatic dependent launch
//   stream_ctas      n         about how many CTAs a weight-streaming product is cut into (0: automatic)
//   stream_min_stages n        stages of the ring a product's CTA is given at least (0: what its k uses; -1: automatic)
//   decode_stages    0, 2..4   stages of keys in flight in decode attention (0: automatic)
//   decode_cluster   0 / 1     merge decode attention's pieces inside a cluster where possible
//   decode_tma       0 / 1     fetch decode attention's keys by bulk tensor copies where possible
//   prefill_splits   0,1,2,4   CTAs that share a tile's keys in the tcgen05 prefill attention (0: automatic)
//   gemm_pair        -1 / 0    two SMs to a tile in the tcgen05 product of many rows (-1: where it applies)
//   filtered_cluster 0 / 1     the cluster kernel of top-k / top-p sampling where the vocabulary fits
extern "C" void rlis_stream_gemm_set_target(int);
extern "C" void rlis_stream_gemm_set_min_stages(int);
extern "C" void rlis_gemm_tcgen05_set_pair(int);
extern "C" void rlis_attention_decode_set_stages(int);
extern "C" void rlis_attention_decode_set_cluster(int);
extern "C" void rlis_attention_decode_set_tma(int);
extern "C" void rlis_attention_prefill_tc_set_splits(int);
extern "C" void rlis_sample_filtered_set_cluster(int);

extern "C" int rlis_debug_set(const char* name, int value) {
    if (name == nullptr) return RLIS_ERR_UNSUPPORTED;
    if (!strcmp(name, "pdl")) rlis_set_pdl(value);
    else if (!strcmp(name, "stream_ctas")) rlis_stream_gemm_set_target(value);
    else if (!strcmp(name, "stream_min_stages")) rlis_stream_gemm_set_min_stages(value);
    else if (!strcmp(name, "decode_stages")) rlis_attention_decode_set_stages(value);
    else if (!strcmp(name, "decode_cluster")) rlis_attention_decode_set_cluster(value);
    else if (!strcmp(name, "decode_tma")) rlis_attention_decode_set_tma(value);
    else if (!strcmp(name, "prefill_splits")) rlis_attention_prefill_tc_set_splits(value);
    else if (!strcmp(name, "gemm_pair")) rlis_gemm_tcgen05_set_pair(value);
    else if (!strcmp(name, "filtered_cluster")) rlis_sample_filtered_set_cluster(value);
    else return RLIS_ERR_UNSUPPORTED;
    return 0;
}

// ---- the error word --------------------------------------------------------------------------
// Each translation unit with bounded waits has an error word of its own on the device.  This
// kernel reads and clears them all and leaves their union in `out`, in stream order, so that an
// engine can bring it to the host with the copy it makes anyway at the end of a step.
extern "C" int* rlis_gemm_tcgen05_error_addr(void);
extern "C" int* rlis_stream_gemm_error_addr(void);
extern "C" int* rlis_attention_prefill_tc_error_addr(void);
extern "C" int* rlis_attention_decode_error_addr(void);

namespace {
struct ErrorWords { int* w[4]; };

__global__ void take_errors_kernel(ErrorWords words, int* __restrict__ out) {
    pdl_wait_and_trigger();
    int v = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) v |= atomicExch(words.w[i], 0);
    *out = v;
}

constexpr int kMaxDevices = 64;
ErrorWords g_words[kMaxDevices];
bool g_words_known[kMaxDevices];
}  // namespace

// out: one int on the device.  The words' addresses are looked up at the first call on a device.
extern "C" int rlis_take_errors(int* out, cudaStream_t stream) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return RLIS_ERR_UNSUPPORTED;
    if (!g_words_known[dev]) {
        ErrorWords w = {{rlis_gemm_tcgen05_error_addr(), rlis_stream_gemm_error_addr(),
                         rlis_attention_prefill_tc_error_addr(), rlis_attention_decode_error_addr()}};
        for (int i = 0; i < 4; ++i)
            if (w.w[i] == nullptr) return RLIS_ERR_UNSUPPORTED;
        g_words[dev] = w;
        g_words_known[dev] = true;
    }
    rlis_launch(take_errors_kernel, dim3(1), dim3(1), 0, stream, g_words[dev], out);
    return RLIS_LAUNCH_CHECK();
}

// Switch for programmatic dependent launch (see common.cuh).
#include "common.cuh"

// On by default: the decode step (batch 8, context 4096, replayed from a graph) measured 1.15 ms
// with it and 1.27 ms without.  What it buys is the weight-streaming product's first requests for
// weights, which go out while the kernel before is still running.
int g_rlis_pdl = 1;

extern "C" void rlis_set_pdl(int on) { g_rlis_pdl = on ? 1 : 0; }
extern "C" int rlis_get_pdl(void) { return g_rlis_pdl; }

// Switch for programmatic dependent launch (see common.cuh).
#include "common.cuh"

// Off by default: inside captured graphs, where the decode step runs, it measured 3-6 % slower
// than plain launches (the graph already removes the launch gaps it is meant to hide).
int g_rlis_pdl = 0;

extern "C" void rlis_set_pdl(int on) { g_rlis_pdl = on ? 1 : 0; }
extern "C" int rlis_get_pdl(void) { return g_rlis_pdl; }

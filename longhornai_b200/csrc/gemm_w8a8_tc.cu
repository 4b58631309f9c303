// placeholder: filled in below
#include "common.cuh"
#include "dispatch.h"
namespace lhb {
bool w8a8_fast_ok(int, int, int) { return false; }
int launch_w8a8_fast(lhb_ctx*, const int8_t*, const int8_t*, const float*, const float*, float*, int,
                     int, int, float, float, cudaStream_t) { return LHB_ERR_UNSUPPORTED; }
}

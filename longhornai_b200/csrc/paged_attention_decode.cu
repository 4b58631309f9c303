// placeholder: filled in below
#include "common.cuh"
#include "dispatch.h"
namespace lhb {
bool decode_fast_ok(const lhb_paged_attn_cfg&, const lhb_paged_layout&) { return false; }
int launch_decode_fast(lhb_ctx*, const float*, const int8_t*, const int8_t*, const float*, const float*,
                       const int32_t*, int, const int32_t*, int, float*, const lhb_paged_attn_cfg&,
                       const lhb_paged_layout&, cudaStream_t) { return LHB_ERR_UNSUPPORTED; }
}

// Shared declarations of the lhb200 library: the context object, error
// plumbing and small device helpers used by every kernel file.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <string>
#include <unordered_map>

#include "lhb200.h"

namespace lhb {

// Per-thread text of the last failing CUDA call (read by lhb_last_error).
void set_last_error(const char* what, cudaError_t err);
void set_last_error_text(const std::string& text);

#define LHB_CUDA(call)                                   \
    do {                                                 \
        cudaError_t _e = (call);                         \
        if (_e != cudaSuccess) {                         \
            ::lhb::set_last_error(#call, _e);            \
            return LHB_ERR_CUDA;                         \
        }                                                \
    } while (0)

#define LHB_LAUNCH_CHECK()                               \
    do {                                                 \
        cudaError_t _e = cudaGetLastError();             \
        if (_e != cudaSuccess) {                         \
            ::lhb::set_last_error("kernel launch", _e);  \
            return LHB_ERR_CUDA;                         \
        }                                                \
    } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }
inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

// 128-byte opaque tensor-map blob (layout-compatible with CUtensorMap).
struct alignas(64) TensorMap { unsigned char bytes[128]; };

}  // namespace lhb

// The context: one per device.  Scratch is carved out linearly per call (calls
// on one context are expected on one stream at a time; concurrent calls that
// use scratch must use separate contexts).
struct lhb_ctx {
    int device = 0;
    int sm_count = 0;
    int sm_limit = 0;                   // > 0: persistent kernels use at most this many SMs (lhb_ctx_set_sm_limit)
    size_t scratch_bytes = 0;
    unsigned char* scratch = nullptr;   // device
    int* status_word = nullptr;         // device, 0 = ok
    int* counters = nullptr;            // device, zero-initialised, self-resetting
    size_t counters_len = 0;
    std::mutex mu;
    // tensor maps keyed by (pointer, dims, box) -- encoding costs microseconds
    std::unordered_map<std::string, lhb::TensorMap> tmaps;
};

namespace lhb {

// Tuning overrides from the environment (LHB_*), read once per process on first use; 0 / -1 = not set.
struct Knobs {
    bool pdl = true;             // LHB_PDL=0: no programmatic dependent launch
    int w4tc_min_m = 9;          // LHB_W4TC_MIN_M: fewest rows that take the W4A16 tensor-core kernel (measured: the GEMV
                                 // kernel needs 31-32 us for 9-16 rows of the 4096 x 14336 shape, this kernel 24 us)
    bool w4tc_stream_k = false;  // LHB_W4TC_SPLIT=1: even deal of units instead of whole CTAs per column tile
    int w4tc_ctas = 0;           // LHB_W4TC_CTAS: cap on its grid
    bool w4tc_coop = true;       // LHB_W4TC_COOP=0: the last CTA to reach a column tile adds its partial sums up alone
    bool w8a8_pair = true;       // LHB_W8A8_PAIR=0: single-CTA W8A8 kernel for every M
    bool w8a8_push_tma = true;   // LHB_W8A8_PUSH=st: sharded W8A8 pushes with plain stores instead of bulk stores
    int gemv_ctas_per_sm = 0;    // LHB_GEMV_CTAS_PER_SM
    int gemv_smem_kb = 0;        // LHB_GEMV_SMEM_KB
    int decode_target = 0;       // LHB_DECODE_TARGET: CTAs per SM the split-KV plan aims at
    int decode_pages = 0;        // LHB_DECODE_PAGES: pages per CTA
    int decode_splits = 0;       // LHB_DECODE_SPLITS: cap on the KV splits
    bool decode_one_wave = true; // LHB_DECODE_ONE_WAVE=0: always aim at four CTAs per SM, also when one wave would hold all items
};
const Knobs& knobs();

// ---------------------------------------------------------------------------
// device helpers
// ---------------------------------------------------------------------------

// Saturating round-half-even to [-lim, lim]; the reference's sat_round_i8 /
// sat_round_i4 / saturate_round (src/kernels/quant.cpp:12-19, :117-124,
// src/kernels/kvcache_quant.cpp:14-23).  NaN maps to -lim, which is what
// lrintf + clamp gives on x86-64.
__device__ __forceinline__ int sat_rne(float v, int lim) {
    const float l = static_cast<float>(lim);
    if (v >= l) return lim;
    if (v <= -l) return -lim;
    if (v != v) return -lim;
    int r = __float2int_rn(v);
    r = r > lim ? lim : r;
    r = r < -lim ? -lim : r;
    return r;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Largest magnitude of four floats as raw bits (sign cleared).  Unlike fmaxf this keeps a NaN
// (bits above 0x7f800000) or an infinity (0x7f800000): a non-finite input wins the maximum.
__device__ __forceinline__ unsigned abs_bits_max4(float4 v) {
    return max(max(__float_as_uint(v.x) & 0x7fffffffu, __float_as_uint(v.y) & 0x7fffffffu),
               max(__float_as_uint(v.z) & 0x7fffffffu, __float_as_uint(v.w) & 0x7fffffffu));
}
// Inverse of the power-of-two digit factor 2^(se-127) for a row whose largest magnitude has the
// bits `mb`; NaN when the row holds a NaN or an infinity, so that every output of the row is NaN
// (the reference's fp32 sums would be NaN or Inf there; finite digits would hide the fault).
__device__ __forceinline__ float digit_inv_scale(unsigned mb, int se) {
    return mb >= 0x7f800000u ? __uint_as_float(0x7fc00000u) : __uint_as_float(static_cast<uint32_t>(254 - se) << 23);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// SwiGLU of one element: (gate * sigmoid(gate)) * value with sigmoid(v) = 1 / (1 + exp(-v)), in the
// reference's operation order (src/kernels/activation.cpp:12, 46-55).
__device__ __forceinline__ float swiglu_one(float g, float v) {
    const float sg = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-g)));
    return __fmul_rn(__fmul_rn(g, sg), v);
}

// sin and cos of the rotary angle of pair i at position p: p * freq_scale / theta_base^(2i/head_dim)
// (src/kernels/rope.cpp:9-15).  The power goes through double precision and is rounded once, as
// the host's powf does: a few ulps in the frequency would become 1e-3 rad at position 8000.
__device__ __forceinline__ void rope_sincos(int p, int i, int head_dim, float theta_base, float freq_scale,
                                            float* sn, float* c) {
    const float pos = __fmul_rn(static_cast<float>(p), freq_scale);
    const float exponent = __fdiv_rn(static_cast<float>(2 * i), static_cast<float>(head_dim));
    const float inv_freq = __fdiv_rn(1.0f, static_cast<float>(pow(static_cast<double>(theta_base),
                                                                   static_cast<double>(exponent))));
    sincosf(__fmul_rn(pos, inv_freq), sn, c);
}

}  // namespace lhb

// Drop-in C++ front end: the reference's `namespace lh` functions for the
// quantized decode path, with the reference's exact signatures, implemented on
// the GPU through the lhb200 C ABI (link liblhb200.so).
//
// Point the include path at include/lh_dropin instead of the reference's src/
// and the same `#include "kernels/gemm_quant.hpp"` lines resolve to these
// declarations (the per-file headers under kernels/ forward here).
//
// Pointer arguments may be host or device pointers, independently of each other:
//   * device pointers are passed straight to the kernels, the call is enqueued
//     on lh::dropin::stream() and returns without synchronising;
//   * host pointers are staged (copied to the device, and results copied back)
//     and the call returns after the results are in host memory, so code written
//     against the reference (all-host buffers) runs unmodified.
// Differences from the reference, which validates nothing and returns void: a
// shape the reference would treat as undefined behaviour, or a CUDA failure,
// throws std::runtime_error.  There is no CPU fallback.
#ifndef LH_DROPIN_HPP
#define LH_DROPIN_HPP

#include <cstdint>

#define LH_DROPIN_API __attribute__((visibility("default")))

namespace lh {

// -- src/kernels/kvcache.hpp:26-41 ------------------------------------------------
struct PagedCacheLayout {
    int num_blocks = 0;
    int block_size = 16;
    int n_kv_heads = 1;
    int head_dim = 1;
};

inline int64_t paged_offset(const PagedCacheLayout& L, int block, int head, int slot, int d) {
    return (((static_cast<int64_t>(block) * L.n_kv_heads + head) * L.block_size + slot) * L.head_dim) + d;
}

// -- src/kernels/kvcache_quant.hpp:31-36 ---------------------------------------------
inline int64_t paged_scale_offset(const PagedCacheLayout& L, int block, int head, int slot) {
    return (static_cast<int64_t>(block) * L.n_kv_heads + head) * L.block_size + slot;
}

// -- src/kernels/paged_attention.hpp:28-37 ---------------------------------------------
struct PagedAttnConfig {
    int n_q_heads = 1;
    int n_kv_heads = 1;
    int seq_q = 1;
    int head_dim = 1;
    bool causal = true;
    float scale = 0.0f;   // <= 0: 1/sqrt(head_dim)
    int window = 0;
    int chunk = 0;
};

// -- src/kernels/dtypes.hpp:305-318 -----------------------------------------------------------
// E4M3 storage byte (4 exponent bits, bias 7; 3 mantissa bits; no infinities, 0x7f / 0xff = NaN;
// largest finite value 448).  Same layout and members as the reference's type, so buffers of it
// are interchangeable; the conversions are host-side helpers (round to nearest even, saturating at
// +-448, NaN and infinities to the NaN code).
namespace dropin {
inline uint8_t float_to_e4m3_bits(float v) {
    uint32_t x;
    static_assert(sizeof(x) == sizeof(v), "float is 32 bits");
    __builtin_memcpy(&x, &v, sizeof x);
    const uint32_t sign = (x >> 24) & 0x80u;
    const int e = static_cast<int>((x >> 23) & 0xff);
    uint32_t m = x & 0x7fffffu;
    if (e == 0xff) return static_cast<uint8_t>(sign | 0x7fu);
    const int ne = e - 120;                               // exponent field of the result
    if (ne > 15 || (ne == 15 && m > 0x600000u)) return static_cast<uint8_t>(sign | 0x7eu);
    uint32_t keep, rest, half_ulp, base = 0;
    if (ne >= 1) {
        keep = m >> 20; rest = m & 0xfffffu; half_ulp = 0x80000u; base = static_cast<uint32_t>(ne) << 3;
    } else {
        if (ne < -2) return static_cast<uint8_t>(sign);
        m |= 0x800000u;
        const int sh = 21 - ne;
        keep = m >> sh; rest = m & ((1u << sh) - 1u); half_ulp = 1u << (sh - 1);
    }
    uint32_t out = base + keep;                           // a mantissa carry runs into the exponent
    if (rest > half_ulp || (rest == half_ulp && (out & 1u))) ++out;
    if (out > 0x7eu) out = 0x7eu;
    return static_cast<uint8_t>(sign | out);
}
inline float e4m3_bits_to_float(uint8_t b) {
    const int e = (b >> 3) & 0xf, m = b & 7;
    uint32_t bits;
    if (e == 0xf && m == 7) bits = 0x7fc00000u;
    else if (e == 0) {
        const float mag = static_cast<float>(m) * 0.001953125f;      // m * 2^-9
        return (b & 0x80u) ? -mag : mag;
    } else bits = (static_cast<uint32_t>(e + 120) << 23) | (static_cast<uint32_t>(m) << 20);
    bits |= (b & 0x80u) ? 0x80000000u : 0u;
    float f;
    __builtin_memcpy(&f, &bits, sizeof f);
    return f;
}
}  // namespace dropin

struct fp8_e4m3 {
    uint8_t bits = 0;

    fp8_e4m3() = default;
    fp8_e4m3(float v) : bits(dropin::float_to_e4m3_bits(v)) {}
    float to_float() const { return dropin::e4m3_bits_to_float(bits); }
    operator float() const { return to_float(); }
    static fp8_e4m3 from_bits(uint8_t b) { fp8_e4m3 v; v.bits = b; return v; }
};
static_assert(sizeof(fp8_e4m3) == 1, "fp8_e4m3 is one byte");

// -- src/kernels/quant.hpp:31-34 --------------------------------------------------------------
LH_DROPIN_API void q8_quantize_per_tensor(const float* src, int8_t* dst, float* scale_out, int64_t n);
LH_DROPIN_API void q8_dequantize_per_tensor(const int8_t* src, float scale, float* dst, int64_t n);

// -- src/kernels/quant.hpp:81-94 --------------------------------------------------------------
LH_DROPIN_API void fp8_quantize_per_tensor(const float* src, fp8_e4m3* dst, float* scale_out, int64_t n);
LH_DROPIN_API void fp8_dequantize_per_tensor(const fp8_e4m3* src, float scale, float* dst, int64_t n);
LH_DROPIN_API void fp8_quantize_per_row(const float* src, fp8_e4m3* dst, float* scales_out, int rows, int dim);
LH_DROPIN_API void fp8_dequantize_per_row(const fp8_e4m3* src, const float* scales, float* dst, int rows, int dim);
LH_DROPIN_API void fp8_quantize_per_col(const float* src, fp8_e4m3* dst, float* scales_out, int rows, int cols);
LH_DROPIN_API void fp8_dequantize_per_col(const fp8_e4m3* src, const float* scales, float* dst, int rows, int cols);

// -- src/kernels/quant.hpp:38-75 ----------------------------------------------------------
LH_DROPIN_API void q8_quantize_per_row(const float* src, int8_t* dst, float* scales_out, int rows, int dim);
LH_DROPIN_API void q8_dequantize_per_row(const int8_t* src, const float* scales, float* dst, int rows, int dim);
LH_DROPIN_API void q8_quantize_per_col(const float* src, int8_t* dst, float* scales_out, int rows, int cols);
LH_DROPIN_API void q8_dequantize_per_col(const int8_t* src, const float* scales, float* dst, int rows, int cols);
LH_DROPIN_API void q4_quantize_groupwise(const float* src, uint8_t* packed, float* scales_out, int K, int N,
                                         int group_size);
LH_DROPIN_API void q4_dequantize_groupwise(const uint8_t* packed, const float* scales, float* dst, int K, int N,
                                           int group_size);
// host-side nibble read (packed must be a host pointer)
inline int8_t q4_get(const uint8_t* packed, int k, int n, int N) {
    const uint8_t b = packed[static_cast<int64_t>(k / 2) * N + n];
    const int nib = (k & 1) ? (b >> 4) : (b & 0x0f);
    return static_cast<int8_t>((nib & 8) ? nib - 16 : nib);
}

// -- src/kernels/gemm_quant.hpp:42-57 ----------------------------------------------------------
LH_DROPIN_API void gemm_w8a8(const int8_t* A_q, const int8_t* B_q, const float* A_scales, const float* B_scales,
                             float* C, int M, int N, int K, float alpha = 1.0f, float beta = 0.0f);
LH_DROPIN_API void gemm_w4a16_groupwise(const float* A, const uint8_t* B_packed, const float* B_scales, float* C,
                                        int M, int N, int K, int group_size, float alpha = 1.0f,
                                        float beta = 0.0f);
// -- src/kernels/gemm_quant.hpp:66-69 ----------------------------------------------------------
LH_DROPIN_API void gemm_fp8_e4m3(const fp8_e4m3* A, const fp8_e4m3* B, float A_scale, float B_scale, float* C,
                                 int M, int N, int K, float alpha = 1.0f, float beta = 0.0f);
// Weight-only int8 per output channel (the reference composes
// q8_dequantize_per_col + gemm; this is the fused call).
LH_DROPIN_API void gemm_w8a16_perchannel(const float* A, const int8_t* B_q, const float* B_scales, float* C,
                                         int M, int N, int K, float alpha = 1.0f, float beta = 0.0f);

// -- src/kernels/kvcache.hpp:50-55, src/kernels/kvcache_quant.hpp:41-57 --------------------------
LH_DROPIN_API void paged_kv_append(float* k_pool, float* v_pool, const float* k_new, const float* v_new,
                                   const int32_t* block_table, const PagedCacheLayout& L, int past_len,
                                   int seq_new);
LH_DROPIN_API void paged_kv_append_q8(int8_t* k_pool, int8_t* v_pool, float* k_scales, float* v_scales,
                                      const float* k_new, const float* v_new, const int32_t* block_table,
                                      const PagedCacheLayout& L, int past_len, int seq_new);
LH_DROPIN_API void paged_attention_q8(const float* Q, const int8_t* K_pool, const int8_t* V_pool,
                                      const float* K_scales, const float* V_scales, const int32_t* block_table,
                                      int seq_len, float* O, const PagedAttnConfig& cfg,
                                      const PagedCacheLayout& L);
// Batched int8 form with the calling convention of paged_attention_batched.
LH_DROPIN_API void paged_attention_q8_batched(const float* Q, const int8_t* K_pool, const int8_t* V_pool,
                                              const float* K_scales, const float* V_scales,
                                              const int32_t* block_tables, int max_blocks_per_req,
                                              const int32_t* seq_lens, int n_requests, float* O,
                                              const PagedAttnConfig& cfg, const PagedCacheLayout& L);

// -- src/kernels/paged_attention.hpp:42-63 ----------------------------------------------------------
LH_DROPIN_API void paged_attention(const float* Q, const float* K_pool, const float* V_pool,
                                   const int32_t* block_table, int seq_len, float* O,
                                   const PagedAttnConfig& cfg, const PagedCacheLayout& L);
LH_DROPIN_API void paged_attention_batched(const float* Q, const float* K_pool, const float* V_pool,
                                           const int32_t* block_tables, int max_blocks_per_req,
                                           const int32_t* seq_lens, int n_requests, float* O,
                                           const PagedAttnConfig& cfg, const PagedCacheLayout& L);

// -- decode-step glue: src/kernels/normalization.hpp:21, rope.hpp:19-21, activation.hpp:34 ---------
// Same arguments as lh::rmsnorm / lh::rope / lh::swiglu, in a namespace of their own: the
// reference's normalization.cpp, rope.cpp and activation.cpp also hold functions outside
// this path and stay in the build, so these names must not collide with theirs.
namespace b200 {
LH_DROPIN_API void rmsnorm(const float* x, const float* gamma, float* y, int rows, int dim, float eps = 1e-5f);
LH_DROPIN_API void rope(float* x, int seq, int n_heads, int head_dim, float theta_base = 10000.0f,
                        float freq_scale = 1.0f, bool interleaved = true, int pos_offset = 0);
LH_DROPIN_API void swiglu(const float* x, float* y, int rows, int dim);
}  // namespace b200

namespace dropin {
// The CUDA stream device-pointer calls are enqueued on (default: the legacy
// default stream) and a blocking wait for it.
LH_DROPIN_API void set_stream(void* cuda_stream);
LH_DROPIN_API void* stream();
LH_DROPIN_API void synchronize();
}  // namespace dropin

}  // namespace lh

#endif  // LH_DROPIN_HPP

// FP8 E4M3 storage: conversion, quantisers, dequantiser and a shape-agnostic GEMM
// (src/kernels/dtypes.hpp:111-196, quant.cpp:176-249, gemm_quant.cpp:87-104).
// The prefill-sized GEMM runs on the tensor cores (gemm_w8a8_tc.cu).
//
// The conversion is the reference's, bit for bit: round to nearest even, saturate
// at +-448 (code 0x7e), NaN and infinities to the single NaN code 0x7f, values
// below half the smallest subnormal to signed zero.  It is written with integer
// operations rather than the toolkit's fp8 intrinsics, whose saturating mode maps
// infinities to the largest finite value instead.
#include "common.cuh"
#include "dispatch.h"

namespace lhb {

__host__ __device__ inline uint8_t f32_to_e4m3_bits(float v) {
#ifdef __CUDA_ARCH__
    const uint32_t x = __float_as_uint(v);
#else
    uint32_t x;
    memcpy(&x, &v, sizeof x);
#endif
    const uint32_t sign = (x >> 24) & 0x80u;
    const int e = static_cast<int>((x >> 23) & 0xff);
    uint32_t m = x & 0x7fffffu;
    if (e == 0xff) return static_cast<uint8_t>(sign | 0x7fu);
    const int ne = e - 120;                               // exponent field of the result, bias 7
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

__device__ __forceinline__ float e4m3_bits_to_f32(uint8_t b) {
    const int e = (b >> 3) & 0xf, m = b & 7;
    if (e == 0xf && m == 7) return __uint_as_float(((b & 0x80u) ? 0x80000000u : 0u) | 0x7fc00000u);
    const float mag = (e == 0) ? static_cast<float>(m) * 0.001953125f               // m * 2^-9
                               : __uint_as_float((static_cast<uint32_t>(e + 120) << 23) | (static_cast<uint32_t>(m) << 20));
    return (b & 0x80u) ? -mag : mag;
}

// ---- quantisers --------------------------------------------------------------------

// max|x| of a slab, merged with atomicMax on the float bits (`out` starts at 0)
__global__ void __launch_bounds__(256)
fp8_absmax_kernel(const float* __restrict__ src, unsigned* __restrict__ out, int64_t n) {
    float m = 0.0f;
    for (int64_t i = blockIdx.x * 256ll + threadIdx.x; i < n; i += gridDim.x * 256ll) m = fmaxf(m, fabsf(src[i]));
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0 && m > 0.0f) atomicMax(out, __float_as_uint(m));
}

// scale[i] = max / 448 (1 if 0), in place over the max|x| values
__global__ void fp8_max_to_scale_kernel(float* __restrict__ scales, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) scales[i] = (scales[i] > 0.0f) ? __fdiv_rn(scales[i], 448.0f) : 1.0f;
}

// q = e4m3(x * (1 / scale)), one scale for everything
__global__ void fp8_quantize_tensor_kernel(const float* __restrict__ src, uint8_t* __restrict__ dst,
                                           const float* __restrict__ scale, int64_t n) {
    const float inv = __fdiv_rn(1.0f, *scale);
    for (int64_t i = blockIdx.x * 256ll + threadIdx.x; i < n; i += gridDim.x * 256ll)
        dst[i] = f32_to_e4m3_bits(__fmul_rn(src[i], inv));
}

// one CTA per row: max|x|, scale = max / 448, q = e4m3(x * (1 / scale))
__global__ void __launch_bounds__(256)
fp8_quantize_per_row_kernel(const float* __restrict__ src, uint8_t* __restrict__ dst, float* __restrict__ scales,
                            int dim) {
    const int64_t row = blockIdx.x;
    const float* x = src + row * dim;
    uint8_t* q = dst + row * dim;
    __shared__ float red[8];
    float m = 0.0f;
    for (int i = threadIdx.x; i < dim; i += 256) m = fmaxf(m, fabsf(x[i]));
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    m = red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) m = fmaxf(m, red[w]);
    const float scale = (m > 0.0f) ? __fdiv_rn(m, 448.0f) : 1.0f;
    const float inv = __fdiv_rn(1.0f, scale);
    for (int i = threadIdx.x; i < dim; i += 256) q[i] = f32_to_e4m3_bits(__fmul_rn(x[i], inv));
    if (threadIdx.x == 0) scales[row] = scale;
}

__global__ void fp8_col_absmax_kernel(const float* __restrict__ src, unsigned* __restrict__ colmax, int rows, int cols,
                                      int rows_per_cta) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    const int r0 = blockIdx.y * rows_per_cta, r1 = min(rows, r0 + rows_per_cta);
    float m = 0.0f;
    for (int r = r0; r < r1; ++r) m = fmaxf(m, fabsf(src[static_cast<int64_t>(r) * cols + c]));
    if (m > 0.0f) atomicMax(colmax + c, __float_as_uint(m));
}

// q = e4m3(x / scale[c])
__global__ void fp8_quantize_cols_kernel(const float* __restrict__ src, uint8_t* __restrict__ dst,
                                         const float* __restrict__ scales, int rows, int cols, int rows_per_cta) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    const float s = scales[c];
    const int r0 = blockIdx.y * rows_per_cta, r1 = min(rows, r0 + rows_per_cta);
    for (int r = r0; r < r1; ++r) {
        const int64_t i = static_cast<int64_t>(r) * cols + c;
        dst[i] = f32_to_e4m3_bits(__fdiv_rn(src[i], s));
    }
}

// mode 0: scales[0]; 1: scales[row]; 2: scales[col]
__global__ void fp8_dequantize_kernel(const uint8_t* __restrict__ src, const float* __restrict__ scales,
                                      float* __restrict__ dst, int64_t total, int cols, int mode) {
    const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (i >= total) return;
    const float s = mode == 0 ? scales[0] : (mode == 1 ? scales[i / cols] : scales[i % cols]);
    dst[i] = __fmul_rn(e4m3_bits_to_f32(src[i]), s);
}

// ---- GEMM, any shape ------------------------------------------------------------------
constexpr int F8_TN = 128, F8_TM = 16, F8_TK = 64;

__global__ void __launch_bounds__(F8_TN)
gemm_fp8_generic_kernel(const uint8_t* __restrict__ A, const uint8_t* __restrict__ B, float combined,
                        float* __restrict__ C, int M, int N, int K, float beta) {
    __shared__ float As[F8_TM][F8_TK];
    const int n = blockIdx.x * F8_TN + threadIdx.x;
    const int m0 = blockIdx.y * F8_TM, mt = min(F8_TM, M - m0);
    float acc[F8_TM];
#pragma unroll
    for (int i = 0; i < F8_TM; ++i) acc[i] = 0.0f;
    for (int k0 = 0; k0 < K; k0 += F8_TK) {
        const int kt = min(F8_TK, K - k0);
        __syncthreads();
        for (int i = threadIdx.x; i < F8_TM * F8_TK; i += F8_TN) {
            const int r = i / F8_TK, c = i % F8_TK;
            As[r][c] = (r < mt && c < kt) ? e4m3_bits_to_f32(A[static_cast<int64_t>(m0 + r) * K + k0 + c]) : 0.0f;
        }
        __syncthreads();
        if (n < N)
            for (int kk = 0; kk < kt; ++kk) {
                const float b = e4m3_bits_to_f32(B[static_cast<int64_t>(k0 + kk) * N + n]);
#pragma unroll
                for (int i = 0; i < F8_TM; ++i) acc[i] = fmaf(As[i][kk], b, acc[i]);
            }
    }
    if (n < N)
        for (int i = 0; i < mt; ++i) {
            float* c = C + static_cast<int64_t>(m0 + i) * N + n;
            const float v = __fmul_rn(combined, acc[i]);
            *c = (beta == 0.0f) ? v : (beta == 1.0f ? __fadd_rn(*c, v) : __fadd_rn(__fmul_rn(*c, beta), v));
        }
}

int launch_fp8_generic(const uint8_t* A, const uint8_t* B, float combined, float* C, int M, int N, int K, float beta,
                       cudaStream_t st) {
    dim3 grid(ceil_div(N, F8_TN), ceil_div(M, F8_TM));
    gemm_fp8_generic_kernel<<<grid, F8_TN, 0, st>>>(A, B, combined, C, M, N, K, beta);
    LHB_LAUNCH_CHECK();
    return LHB_OK;
}

}  // namespace lhb

using namespace lhb;

#define REQUIRE(cond, code) \
    do {                    \
        if (!(cond)) return (code); \
    } while (0)

extern "C" {

int lhb_fp8_quantize_per_tensor(lhb_ctx* ctx, const float* src, uint8_t* dst, float* scale_out, int64_t n,
                                void* stream) {
    REQUIRE(ctx && src && dst && scale_out, LHB_ERR_NULL);
    REQUIRE(n >= 0, LHB_ERR_BAD_SHAPE);
    cudaStream_t st = as_stream(stream);
    LHB_CUDA(cudaMemsetAsync(scale_out, 0, sizeof(float), st));          // doubles as the max|x| accumulator
    const unsigned grid = static_cast<unsigned>(std::min<int64_t>(std::max<int64_t>(1, ceil_div64(n, 1024)), 2368));
    if (n > 0) {
        fp8_absmax_kernel<<<grid, 256, 0, st>>>(src, reinterpret_cast<unsigned*>(scale_out), n);
        LHB_LAUNCH_CHECK();
    }
    fp8_max_to_scale_kernel<<<1, 32, 0, st>>>(scale_out, 1);
    LHB_LAUNCH_CHECK();
    if (n > 0) {
        fp8_quantize_tensor_kernel<<<grid, 256, 0, st>>>(src, dst, scale_out, n);
        LHB_LAUNCH_CHECK();
    }
    return LHB_OK;
}

int lhb_fp8_quantize_per_row(lhb_ctx* ctx, const float* src, uint8_t* dst, float* scales_out, int rows, int dim,
                             void* stream) {
    REQUIRE(ctx && src && dst && scales_out, LHB_ERR_NULL);
    REQUIRE(rows >= 0 && dim > 0, LHB_ERR_BAD_SHAPE);
    if (rows == 0) return LHB_OK;
    fp8_quantize_per_row_kernel<<<rows, 256, 0, as_stream(stream)>>>(src, dst, scales_out, dim);
    LHB_LAUNCH_CHECK();
    return LHB_OK;
}

int lhb_fp8_quantize_per_col(lhb_ctx* ctx, const float* src, uint8_t* dst, float* scales_out, int rows, int cols,
                             void* stream) {
    REQUIRE(ctx && src && dst && scales_out, LHB_ERR_NULL);
    REQUIRE(rows >= 0 && cols > 0, LHB_ERR_BAD_SHAPE);
    cudaStream_t st = as_stream(stream);
    LHB_CUDA(cudaMemsetAsync(scales_out, 0, sizeof(float) * static_cast<size_t>(cols), st));
    const int rpc = 128;
    dim3 grid(ceil_div(cols, 128), rows > 0 ? ceil_div(rows, rpc) : 1);
    if (rows > 0) {
        fp8_col_absmax_kernel<<<grid, 128, 0, st>>>(src, reinterpret_cast<unsigned*>(scales_out), rows, cols, rpc);
        LHB_LAUNCH_CHECK();
    }
    fp8_max_to_scale_kernel<<<ceil_div(cols, 256), 256, 0, st>>>(scales_out, cols);
    LHB_LAUNCH_CHECK();
    if (rows > 0) {
        fp8_quantize_cols_kernel<<<grid, 128, 0, st>>>(src, dst, scales_out, rows, cols, rpc);
        LHB_LAUNCH_CHECK();
    }
    return LHB_OK;
}

int lhb_fp8_dequantize(lhb_ctx* ctx, const uint8_t* src, const float* scales, float* dst, int rows, int cols,
                       int mode, void* stream) {
    REQUIRE(ctx && src && scales && dst, LHB_ERR_NULL);
    REQUIRE(rows >= 0 && cols > 0 && mode >= 0 && mode <= 2, LHB_ERR_BAD_SHAPE);
    const int64_t total = static_cast<int64_t>(rows) * cols;
    if (total == 0) return LHB_OK;
    fp8_dequantize_kernel<<<static_cast<unsigned>(ceil_div64(total, 256)), 256, 0, as_stream(stream)>>>(
        src, scales, dst, total, cols, mode);
    LHB_LAUNCH_CHECK();
    return LHB_OK;
}

int lhb_gemm_fp8_fast_path(int M, int N, int K) { return w8a8_fast_ok(M, N, K) ? 1 : 0; }

int lhb_gemm_fp8_e4m3(lhb_ctx* ctx, const uint8_t* A, const uint8_t* B, float A_scale, float B_scale, float* C, int M,
                      int N, int K, float alpha, float beta, void* stream) {
    REQUIRE(ctx && A && B && C, LHB_ERR_NULL);
    REQUIRE(M >= 0 && N > 0 && K > 0, LHB_ERR_BAD_SHAPE);
    if (M == 0) return LHB_OK;
    const float combined = alpha * A_scale * B_scale;       // the reference's order (gemm_quant.cpp:91)
    cudaStream_t st = as_stream(stream);
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (w8a8_fast_ok(M, N, K) && al16(A) && al16(B) && al16(C))
        return launch_fp8_fast(ctx, A, B, combined, C, M, N, K, beta, st);
    return launch_fp8_generic(A, B, combined, C, M, N, K, beta, st);
}

}  // extern "C"

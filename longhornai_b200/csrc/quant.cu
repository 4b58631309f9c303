// Quantisers and dequantisers, bit-exact with the reference.
//
// Two idioms coexist in the reference and both are kept verbatim with IEEE
// round-to-nearest intrinsics (no FMA contraction, no fast-math):
//   reciprocal multiply  q = sat(x * (1/scale))   per-row int8 (quant.cpp:52-63)
//   true division        q = sat(x / scale)       per-col int8 (quant.cpp:75-96),
//                                                 int4 groups  (quant.cpp:128-160)
// max|x| reductions are order-independent (max is exact), so a parallel
// reduction gives the same scale as the serial loop.
//
// All kernels here are HBM-bound streaming passes; they are offline (weights)
// or small (activations) next to the GEMMs they feed.
#include <algorithm>

#include "common.cuh"

namespace lhb {

// ---- int8 per row ----------------------------------------------------------

// One CTA per row: pass 1 max|x| (block reduce), pass 2 quantise (the row is
// re-read from L1/L2).
__global__ void __launch_bounds__(256)
q8_quantize_per_row_kernel(const float* __restrict__ src, int8_t* __restrict__ dst,
                           float* __restrict__ scales, int dim) {
    const int64_t row = blockIdx.x;
    const float* x = src + row * dim;
    int8_t* q = dst + row * dim;
    __shared__ float red[8];
    float m = 0.0f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) m = fmaxf(m, fabsf(x[i]));
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    m = red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) m = fmaxf(m, red[w]);
    const float scale = (m > 0.0f) ? __fdiv_rn(m, 127.0f) : 1.0f;
    const float inv = __fdiv_rn(1.0f, scale);
    for (int i = threadIdx.x; i < dim; i += blockDim.x)
        q[i] = static_cast<int8_t>(sat_rne(__fmul_rn(x[i], inv), 127));
    if (threadIdx.x == 0) scales[row] = scale;
}

__global__ void q8_dequantize_per_row_kernel(const int8_t* __restrict__ src,
                                             const float* __restrict__ scales,
                                             float* __restrict__ dst, int64_t total, int dim) {
    const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (i < total) dst[i] = __fmul_rn(static_cast<float>(src[i]), scales[i / dim]);
}

// ---- int8 per tensor -----------------------------------------------------------
// (src/kernels/quant.cpp:33-49: one scale = max|x| / 127, reciprocal-multiply idiom as per row.)
// Three small passes: max|x| merged with atomicMax on the float bits into the scale word itself,
// bits -> scale, quantise.

__global__ void __launch_bounds__(256)
tensor_absmax_kernel(const float* __restrict__ src, unsigned* __restrict__ maxbits, int64_t n) {
    float m = 0.0f;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x)
        m = fmaxf(m, fabsf(src[i]));
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0 && m > 0.0f) atomicMax(maxbits, __float_as_uint(m));
}

__global__ void q8_max_to_scale_kernel(float* scale) {
    const float m = *scale;                       // holds max|x| (its bits were merged as unsigned)
    *scale = (m > 0.0f) ? __fdiv_rn(m, 127.0f) : 1.0f;
}

__global__ void __launch_bounds__(256)
q8_quantize_tensor_kernel(const float* __restrict__ src, int8_t* __restrict__ dst, const float* __restrict__ scale,
                          int64_t n) {
    const float inv = __fdiv_rn(1.0f, *scale);
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x)
        dst[i] = static_cast<int8_t>(sat_rne(__fmul_rn(src[i], inv), 127));
}

__global__ void q8_dequantize_tensor_kernel(const int8_t* __restrict__ src, float scale, float* __restrict__ dst,
                                            int64_t n) {
    const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (i < n) dst[i] = __fmul_rn(static_cast<float>(src[i]), scale);
}

// ---- int8 per column ---------------------------------------------------------

// Column max|x| over a slab of rows, merged with atomicMax on the float bits
// (non-negative floats order like unsigned integers).  `colmax` starts at 0.
__global__ void col_absmax_kernel(const float* __restrict__ src, unsigned* __restrict__ colmax,
                                  int rows, int cols, int rows_per_cta) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    const int r0 = blockIdx.y * rows_per_cta;
    const int r1 = min(rows, r0 + rows_per_cta);
    float m = 0.0f;
    for (int r = r0; r < r1; ++r) m = fmaxf(m, fabsf(src[static_cast<int64_t>(r) * cols + c]));
    if (m > 0.0f) atomicMax(colmax + c, __float_as_uint(m));
}

__global__ void absmax_to_scale_kernel(float* __restrict__ scales, int n, float qmax) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const float m = scales[i];
        scales[i] = (m > 0.0f) ? __fdiv_rn(m, qmax) : 1.0f;
    }
}

__global__ void q8_quantize_cols_kernel(const float* __restrict__ src, int8_t* __restrict__ dst,
                                        const float* __restrict__ scales, int rows, int cols,
                                        int rows_per_cta) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    const float s = scales[c];
    const int r0 = blockIdx.y * rows_per_cta;
    const int r1 = min(rows, r0 + rows_per_cta);
    for (int r = r0; r < r1; ++r) {
        const int64_t i = static_cast<int64_t>(r) * cols + c;
        dst[i] = static_cast<int8_t>(sat_rne(__fdiv_rn(src[i], s), 127));
    }
}

__global__ void q8_dequantize_per_col_kernel(const int8_t* __restrict__ src,
                                             const float* __restrict__ scales,
                                             float* __restrict__ dst, int64_t total, int cols) {
    const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (i < total) dst[i] = __fmul_rn(static_cast<float>(src[i]), scales[i % cols]);
}

// ---- int4 group-wise ------------------------------------------------------------

// scale[g, n] = max|w[gG..gG+G, n]| / 7, one thread per (g, n).
__global__ void q4_group_scale_kernel(const float* __restrict__ src, float* __restrict__ scales,
                                      int N, int G) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= N) return;
    const int g = blockIdx.y;
    const float* p = src + static_cast<int64_t>(g) * G * N + n;
    float m = 0.0f;
    for (int k = 0; k < G; ++k) m = fmaxf(m, fabsf(p[static_cast<int64_t>(k) * N]));
    scales[static_cast<int64_t>(g) * N + n] = (m > 0.0f) ? __fdiv_rn(m, 7.0f) : 1.0f;
}

// One thread per packed byte: rows 2r (low nibble) and 2r+1 (high nibble).
__global__ void q4_pack_kernel(const float* __restrict__ src, const float* __restrict__ scales,
                               uint8_t* __restrict__ packed, int K, int N, int G) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= N) return;
    const int k = 2 * blockIdx.y;
    const float s0 = scales[static_cast<int64_t>(k / G) * N + n];
    const float s1 = scales[static_cast<int64_t>((k + 1) / G) * N + n];
    const int lo = sat_rne(__fdiv_rn(src[static_cast<int64_t>(k) * N + n], s0), 7);
    const int hi = sat_rne(__fdiv_rn(src[static_cast<int64_t>(k + 1) * N + n], s1), 7);
    packed[static_cast<int64_t>(k >> 1) * N + n] =
        static_cast<uint8_t>((lo & 0xf) | ((hi & 0xf) << 4));
}

__global__ void q4_dequantize_kernel(const uint8_t* __restrict__ packed,
                                     const float* __restrict__ scales, float* __restrict__ dst,
                                     int K, int N, int G) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= N) return;
    const int k = blockIdx.y;
    const uint8_t b = packed[static_cast<int64_t>(k >> 1) * N + n];
    int nib = (k & 1) ? (b >> 4) : (b & 0xf);
    nib = (nib & 8) ? nib - 16 : nib;
    dst[static_cast<int64_t>(k) * N + n] =
        __fmul_rn(static_cast<float>(nib), scales[static_cast<int64_t>(k / G) * N + n]);
}

}  // namespace lhb

using namespace lhb;

#define REQUIRE(cond, code) \
    do {                    \
        if (!(cond)) return (code); \
    } while (0)

extern "C" {

int lhb_q8_quantize_per_tensor(lhb_ctx* ctx, const float* src, int8_t* dst, float* scale_out, int64_t n,
                               void* stream) {
    REQUIRE(ctx && src && dst && scale_out, LHB_ERR_NULL);
    REQUIRE(n >= 0, LHB_ERR_BAD_SHAPE);
    cudaStream_t st = as_stream(stream);
    LHB_CUDA(cudaMemsetAsync(scale_out, 0, sizeof(float), st));          // doubles as the max|x| accumulator
    const unsigned grid = static_cast<unsigned>(std::min<int64_t>(std::max<int64_t>(1, ceil_div64(n, 1024)), 2368));
    if (n > 0) {
        tensor_absmax_kernel<<<grid, 256, 0, st>>>(src, reinterpret_cast<unsigned*>(scale_out), n);
        LHB_LAUNCH_CHECK();
    }
    q8_max_to_scale_kernel<<<1, 1, 0, st>>>(scale_out);
    LHB_LAUNCH_CHECK();
    if (n > 0) {
        q8_quantize_tensor_kernel<<<grid, 256, 0, st>>>(src, dst, scale_out, n);
        LHB_LAUNCH_CHECK();
    }
    return LHB_OK;
}

int lhb_q8_dequantize_per_tensor(lhb_ctx* ctx, const int8_t* src, float scale, float* dst, int64_t n, void* stream) {
    REQUIRE(ctx && src && dst, LHB_ERR_NULL);
    REQUIRE(n >= 0, LHB_ERR_BAD_SHAPE);
    if (n == 0) return LHB_OK;
    q8_dequantize_tensor_kernel<<<static_cast<unsigned>(ceil_div64(n, 256)), 256, 0, as_stream(stream)>>>(src, scale,
                                                                                                          dst, n);
    LHB_LAUNCH_CHECK();
    return LHB_OK;
}

int lhb_q8_quantize_per_row(lhb_ctx* ctx, const float* src, int8_t* dst, float* scales_out,
                            int rows, int dim, void* stream) {
    REQUIRE(ctx && src && dst && scales_out, LHB_ERR_NULL);
    REQUIRE(rows >= 0 && dim > 0, LHB_ERR_BAD_SHAPE);
    if (rows == 0) return LHB_OK;
    q8_quantize_per_row_kernel<<<rows, 256, 0, as_stream(stream)>>>(src, dst, scales_out, dim);
    LHB_LAUNCH_CHECK();
    return LHB_OK;
}

int lhb_q8_dequantize_per_row(lhb_ctx* ctx, const int8_t* src, const float* scales, float* dst,
                              int rows, int dim, void* stream) {
    REQUIRE(ctx && src && dst && scales, LHB_ERR_NULL);
    REQUIRE(rows >= 0 && dim > 0, LHB_ERR_BAD_SHAPE);
    const int64_t total = static_cast<int64_t>(rows) * dim;
    if (total == 0) return LHB_OK;
    q8_dequantize_per_row_kernel<<<static_cast<unsigned>(ceil_div64(total, 256)), 256, 0,
                                   as_stream(stream)>>>(src, scales, dst, total, dim);
    LHB_LAUNCH_CHECK();
    return LHB_OK;
}

int lhb_q8_quantize_per_col(lhb_ctx* ctx, const float* src, int8_t* dst, float* scales_out,
                            int rows, int cols, void* stream) {
    REQUIRE(ctx && src && dst && scales_out, LHB_ERR_NULL);
    REQUIRE(rows >= 0 && cols > 0, LHB_ERR_BAD_SHAPE);
    cudaStream_t st = as_stream(stream);
    // scales_out doubles as the max|x| accumulator (float bits, starts at 0)
    LHB_CUDA(cudaMemsetAsync(scales_out, 0, sizeof(float) * static_cast<size_t>(cols), st));
    const int rpc = 128;
    dim3 grid(ceil_div(cols, 128), rows > 0 ? ceil_div(rows, rpc) : 1);
    if (rows > 0) {
        col_absmax_kernel<<<grid, 128, 0, st>>>(src, reinterpret_cast<unsigned*>(scales_out), rows,
                                                cols, rpc);
        LHB_LAUNCH_CHECK();
    }
    absmax_to_scale_kernel<<<ceil_div(cols, 256), 256, 0, st>>>(scales_out, cols, 127.0f);
    LHB_LAUNCH_CHECK();
    if (rows > 0) {
        q8_quantize_cols_kernel<<<grid, 128, 0, st>>>(src, dst, scales_out, rows, cols, rpc);
        LHB_LAUNCH_CHECK();
    }
    return LHB_OK;
}

int lhb_q8_dequantize_per_col(lhb_ctx* ctx, const int8_t* src, const float* scales, float* dst,
                              int rows, int cols, void* stream) {
    REQUIRE(ctx && src && dst && scales, LHB_ERR_NULL);
    REQUIRE(rows >= 0 && cols > 0, LHB_ERR_BAD_SHAPE);
    const int64_t total = static_cast<int64_t>(rows) * cols;
    if (total == 0) return LHB_OK;
    q8_dequantize_per_col_kernel<<<static_cast<unsigned>(ceil_div64(total, 256)), 256, 0,
                                   as_stream(stream)>>>(src, scales, dst, total, cols);
    LHB_LAUNCH_CHECK();
    return LHB_OK;
}

int lhb_q4_quantize_groupwise(lhb_ctx* ctx, const float* src, uint8_t* packed, float* scales_out,
                              int K, int N, int group_size, void* stream) {
    REQUIRE(ctx && src && packed && scales_out, LHB_ERR_NULL);
    REQUIRE(K > 0 && N > 0 && group_size > 0, LHB_ERR_BAD_SHAPE);
    REQUIRE((K % 2) == 0 && (K % group_size) == 0, LHB_ERR_BAD_SHAPE);
    REQUIRE(K / 2 <= 65535, LHB_ERR_UNSUPPORTED);  // grid.y limit
    cudaStream_t st = as_stream(stream);
    q4_group_scale_kernel<<<dim3(ceil_div(N, 128), K / group_size), 128, 0, st>>>(src, scales_out,
                                                                                 N, group_size);
    LHB_LAUNCH_CHECK();
    q4_pack_kernel<<<dim3(ceil_div(N, 128), K / 2), 128, 0, st>>>(src, scales_out, packed, K, N,
                                                                 group_size);
    LHB_LAUNCH_CHECK();
    return LHB_OK;
}

int lhb_q4_dequantize_groupwise(lhb_ctx* ctx, const uint8_t* packed, const float* scales,
                                float* dst, int K, int N, int group_size, void* stream) {
    REQUIRE(ctx && packed && scales && dst, LHB_ERR_NULL);
    REQUIRE(K > 0 && N > 0 && group_size > 0, LHB_ERR_BAD_SHAPE);
    REQUIRE((K % 2) == 0 && (K % group_size) == 0, LHB_ERR_BAD_SHAPE);
    REQUIRE(K <= 65535, LHB_ERR_UNSUPPORTED);
    q4_dequantize_kernel<<<dim3(ceil_div(N, 128), K), 128, 0, as_stream(stream)>>>(
        packed, scales, dst, K, N, group_size);
    LHB_LAUNCH_CHECK();
    return LHB_OK;
}

}  // extern "C"

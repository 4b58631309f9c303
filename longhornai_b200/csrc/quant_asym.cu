// Asymmetric int4 with fp16 scale and zero-point per group: quantiser, dequantiser
// and a shape-agnostic GEMM.  An extension of the reference's symmetric int4
// (src/kernels/quant.hpp:52-57): same packing - byte (k/2, n), low nibble = even
// k - but the nibble is unsigned, u in [0, 15], and each group of G rows of a
// column carries an fp16 scale and an fp16 (integer-valued) zero-point:
//   lo = min(0, min w), hi = max(0, max w);  s = fp16((hi - lo) / 15), 1 if 0
//   z = clamp(rint(-lo / s), 0, 15);  u = clamp(rint(w / s) + z, 0, 15)
//   w' = (u - z) * s
// Arithmetic uses IEEE round-to-nearest intrinsics throughout, so packed bytes
// and parameters are bit-identical to the CPU statement of the same rules.
// The fast path for decode shapes lives in gemv_mma.cu.
#include <cuda_fp16.h>

#include "common.cuh"
#include "dispatch.h"

namespace lhb {

__device__ __forceinline__ float h2f_bits(uint16_t b) { return __half2float(__ushort_as_half(b)); }
__device__ __forceinline__ uint16_t f2h_bits(float v) { return __half_as_ushort(__float2half_rn(v)); }

// one thread per (group, column)
__global__ void q4a_group_params_kernel(const float* __restrict__ src, uint16_t* __restrict__ scales_h,
                                        uint16_t* __restrict__ zeros_h, int N, int G) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= N) return;
    const int g = blockIdx.y;
    const float* p = src + static_cast<int64_t>(g) * G * N + n;
    float lo = 0.0f, hi = 0.0f;
    for (int k = 0; k < G; ++k) {
        const float w = p[static_cast<int64_t>(k) * N];
        lo = fminf(lo, w);
        hi = fmaxf(hi, w);
    }
    float s = h2f_bits(f2h_bits(__fdiv_rn(__fsub_rn(hi, lo), 15.0f)));
    if (!(s > 0.0f)) s = 1.0f;
    const int z = min(15, max(0, __float2int_rn(__fdiv_rn(-lo, s))));
    scales_h[static_cast<int64_t>(g) * N + n] = f2h_bits(s);
    zeros_h[static_cast<int64_t>(g) * N + n] = f2h_bits(static_cast<float>(z));
}

// one thread per packed byte: rows 2r (low nibble) and 2r + 1 (high nibble)
__global__ void q4a_pack_kernel(const float* __restrict__ src, const uint16_t* __restrict__ scales_h,
                                const uint16_t* __restrict__ zeros_h, uint8_t* __restrict__ packed, int K, int N,
                                int G) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    const int r = blockIdx.y;
    if (n >= N) return;
    uint32_t byte = 0;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int k = 2 * r + half, g = k / G;
        const float s = h2f_bits(scales_h[static_cast<int64_t>(g) * N + n]);
        const int z = static_cast<int>(h2f_bits(zeros_h[static_cast<int64_t>(g) * N + n]));
        const int u = min(15, max(0, __float2int_rn(__fdiv_rn(src[static_cast<int64_t>(k) * N + n], s)) + z));
        byte |= static_cast<uint32_t>(u) << (4 * half);
    }
    packed[static_cast<int64_t>(r) * N + n] = static_cast<uint8_t>(byte);
}

__global__ void q4a_dequantize_kernel(const uint8_t* __restrict__ packed, const uint16_t* __restrict__ scales_h,
                                      const uint16_t* __restrict__ zeros_h, float* __restrict__ dst, int64_t total,
                                      int N, int G) {
    const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (i >= total) return;
    const int k = static_cast<int>(i / N), n = static_cast<int>(i % N), g = k / G;
    const uint8_t b = packed[static_cast<int64_t>(k >> 1) * N + n];
    const int u = (k & 1) ? (b >> 4) : (b & 0xf);
    const int z = static_cast<int>(h2f_bits(zeros_h[static_cast<int64_t>(g) * N + n]));
    dst[i] = __fmul_rn(static_cast<float>(u - z), h2f_bits(scales_h[static_cast<int64_t>(g) * N + n]));
}

// Any shape: one thread per output column, a 16-row strip of A staged through shared
// memory; out[m][n] = sum_g s[g][n] * sum_{k in g} A[m][k] * (u[k][n] - z[g][n]).
constexpr int QA_TN = 128, QA_TM = 16, QA_TK = 64;

__global__ void __launch_bounds__(QA_TN)
gemm_w4a16_asym_generic_kernel(const float* __restrict__ A, const uint8_t* __restrict__ Bp,
                               const uint16_t* __restrict__ scales_h, const uint16_t* __restrict__ zeros_h,
                               float* __restrict__ C, int M, int N, int K, int G, float alpha, float beta) {
    __shared__ float As[QA_TM][QA_TK];
    const int n = blockIdx.x * QA_TN + threadIdx.x;
    const int m0 = blockIdx.y * QA_TM;
    const int mt = min(QA_TM, M - m0);
    float out[QA_TM], acc[QA_TM];
#pragma unroll
    for (int i = 0; i < QA_TM; ++i) out[i] = acc[i] = 0.0f;
    int cur_g = 0;
    float z = (n < N) ? h2f_bits(zeros_h[n]) : 0.0f;
    for (int k0 = 0; k0 < K; k0 += QA_TK) {
        const int kt = min(QA_TK, K - k0);
        __syncthreads();
        for (int i = threadIdx.x; i < QA_TM * QA_TK; i += QA_TN) {
            const int r = i / QA_TK, c = i % QA_TK;
            As[r][c] = (r < mt && c < kt) ? A[static_cast<int64_t>(m0 + r) * K + k0 + c] : 0.0f;
        }
        __syncthreads();
        if (n < N) {
            for (int kk = 0; kk < kt; ++kk) {
                const int k = k0 + kk, g = k / G;
                if (g != cur_g) {
                    const float s = h2f_bits(scales_h[static_cast<int64_t>(cur_g) * N + n]);
#pragma unroll
                    for (int i = 0; i < QA_TM; ++i) { out[i] = fmaf(s, acc[i], out[i]); acc[i] = 0.0f; }
                    cur_g = g;
                    z = h2f_bits(zeros_h[static_cast<int64_t>(g) * N + n]);
                }
                const uint8_t b = Bp[static_cast<int64_t>(k >> 1) * N + n];
                const float q = static_cast<float>((k & 1) ? (b >> 4) : (b & 0xf)) - z;
#pragma unroll
                for (int i = 0; i < QA_TM; ++i) acc[i] = fmaf(As[i][kk], q, acc[i]);
            }
        }
    }
    if (n < N) {
        const float s = h2f_bits(scales_h[static_cast<int64_t>(cur_g) * N + n]);
        for (int i = 0; i < mt; ++i) {
            float* c = C + static_cast<int64_t>(m0 + i) * N + n;
            const float v = alpha * fmaf(s, acc[i], out[i]);
            *c = (beta == 0.0f) ? v : fmaf(beta, *c, v);
        }
    }
}

int launch_w4a16_asym_generic(const float* A, const uint8_t* Bp, const uint16_t* Bs, const uint16_t* Bz, float* C,
                              int M, int N, int K, int G, float alpha, float beta, cudaStream_t st) {
    dim3 grid(ceil_div(N, QA_TN), ceil_div(M, QA_TM));
    gemm_w4a16_asym_generic_kernel<<<grid, QA_TN, 0, st>>>(A, Bp, Bs, Bz, C, M, N, K, G, alpha, beta);
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

int lhb_q4a_quantize_groupwise(lhb_ctx* ctx, const float* src, uint8_t* packed, uint16_t* scales_h,
                               uint16_t* zeros_h, int K, int N, int group_size, void* stream) {
    REQUIRE(ctx && src && packed && scales_h && zeros_h, LHB_ERR_NULL);
    REQUIRE(K > 0 && N > 0 && group_size > 0, LHB_ERR_BAD_SHAPE);
    REQUIRE((K % 2) == 0 && (K % group_size) == 0, LHB_ERR_BAD_SHAPE);
    REQUIRE(K / 2 <= 65535, LHB_ERR_UNSUPPORTED);  // grid.y limit
    cudaStream_t st = as_stream(stream);
    q4a_group_params_kernel<<<dim3(ceil_div(N, 128), K / group_size), 128, 0, st>>>(src, scales_h, zeros_h, N,
                                                                                   group_size);
    LHB_LAUNCH_CHECK();
    q4a_pack_kernel<<<dim3(ceil_div(N, 128), K / 2), 128, 0, st>>>(src, scales_h, zeros_h, packed, K, N, group_size);
    LHB_LAUNCH_CHECK();
    return LHB_OK;
}

int lhb_q4a_dequantize_groupwise(lhb_ctx* ctx, const uint8_t* packed, const uint16_t* scales_h,
                                 const uint16_t* zeros_h, float* dst, int K, int N, int group_size, void* stream) {
    REQUIRE(ctx && packed && scales_h && zeros_h && dst, LHB_ERR_NULL);
    REQUIRE(K > 0 && N > 0 && group_size > 0 && (K % 2) == 0 && (K % group_size) == 0, LHB_ERR_BAD_SHAPE);
    const int64_t total = static_cast<int64_t>(K) * N;
    q4a_dequantize_kernel<<<static_cast<unsigned>(ceil_div64(total, 256)), 256, 0, as_stream(stream)>>>(
        packed, scales_h, zeros_h, dst, total, N, group_size);
    LHB_LAUNCH_CHECK();
    return LHB_OK;
}

int lhb_gemm_w4a16_asym_fast_path(int M, int N, int K, int G) { return w4a16_asym_fast_ok(M, N, K, G) ? 1 : 0; }

int lhb_gemm_w4a16_asym(lhb_ctx* ctx, const float* A, const uint8_t* Bp, const uint16_t* scales_h,
                        const uint16_t* zeros_h, float* C, int M, int N, int K, int group_size, float alpha,
                        float beta, void* stream) {
    REQUIRE(ctx && A && Bp && scales_h && zeros_h && C, LHB_ERR_NULL);
    REQUIRE(M >= 0 && N > 0 && K > 0 && group_size > 0, LHB_ERR_BAD_SHAPE);
    REQUIRE((K % 2) == 0 && (K % group_size) == 0, LHB_ERR_BAD_SHAPE);
    if (M == 0) return LHB_OK;
    cudaStream_t st = as_stream(stream);
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (w4a16_asym_fast_ok(M, N, K, group_size) && al16(A) && al16(Bp) && al16(scales_h) && al16(zeros_h) && al16(C))
        return launch_w4a16_asym_fast(ctx, A, Bp, scales_h, zeros_h, C, M, N, K, group_size, alpha, beta, st);
    return launch_w4a16_asym_generic(A, Bp, scales_h, zeros_h, C, M, N, K, group_size, alpha, beta, st);
}

}  // extern "C"

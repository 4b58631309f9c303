// Generic (any-shape) quantized GEMM kernels on the CUDA cores.
//
// These are the safety net behind the tensor-core paths: they accept every
// shape the reference accepts (odd N, group sizes that are not multiples of
// 16, tiny test shapes) and give results within the library tolerance
// (1e-3 relative / 1e-4 absolute against the reference).  One thread owns one
// output column, a CTA owns 128 columns x up to 8 rows of A staged in shared
// memory; weights stream down K with loads coalesced along N.
#include "common.cuh"

namespace lhb {

constexpr int GEN_TN = 128;   // columns per CTA (one per thread)
constexpr int GEN_TM = 8;     // rows of A per CTA
constexpr int GEN_TK = 256;   // K chunk staged in shared memory

// C = beta*C + alpha*acc with the reference's special case: beta == 0 never
// reads C (src/kernels/gemm_quant.cpp:12-21).
__device__ __forceinline__ void store_c(float* c, float acc, float alpha, float beta) {
    *c = (beta == 0.0f) ? alpha * acc : fmaf(beta, *c, alpha * acc);
}

// W4A16 group-wise: out[m][n] = sum_g scale[g][n] * sum_{k in g} A[m][k]*q[k][n].
// Follows src/kernels/gemm_quant.cpp:54-82 up to the order of the fp32 sums.
__global__ void __launch_bounds__(GEN_TN)
gemm_w4a16_generic_kernel(const float* __restrict__ A, const uint8_t* __restrict__ Bp,
                          const float* __restrict__ Bs, float* __restrict__ C, int M, int N,
                          int K, int G, float alpha, float beta) {
    __shared__ float As[GEN_TM][GEN_TK];
    const int n = blockIdx.x * GEN_TN + threadIdx.x;
    const int m0 = blockIdx.y * GEN_TM;
    const int mt = min(GEN_TM, M - m0);
    float out[GEN_TM], acc[GEN_TM];
#pragma unroll
    for (int i = 0; i < GEN_TM; ++i) out[i] = acc[i] = 0.0f;
    int cur_g = 0;
    for (int k0 = 0; k0 < K; k0 += GEN_TK) {
        const int kt = min(GEN_TK, K - k0);
        __syncthreads();
        for (int i = threadIdx.x; i < GEN_TM * GEN_TK; i += GEN_TN) {
            const int r = i / GEN_TK, c = i % GEN_TK;
            As[r][c] = (r < mt && c < kt) ? A[static_cast<int64_t>(m0 + r) * K + k0 + c] : 0.0f;
        }
        __syncthreads();
        if (n < N) {
            for (int kk = 0; kk < kt; ++kk) {
                const int k = k0 + kk;
                const int g = k / G;
                if (g != cur_g) {
                    const float s = Bs[static_cast<int64_t>(cur_g) * N + n];
#pragma unroll
                    for (int i = 0; i < GEN_TM; ++i) { out[i] = fmaf(s, acc[i], out[i]); acc[i] = 0.0f; }
                    cur_g = g;
                }
                const uint8_t b = Bp[static_cast<int64_t>(k >> 1) * N + n];
                int nib = (k & 1) ? (b >> 4) : (b & 0xf);
                nib = (nib & 8) ? nib - 16 : nib;
                const float q = static_cast<float>(nib);
#pragma unroll
                for (int i = 0; i < GEN_TM; ++i) acc[i] = fmaf(As[i][kk], q, acc[i]);
            }
        }
    }
    if (n < N) {
        const float s = Bs[static_cast<int64_t>(cur_g) * N + n];
        for (int i = 0; i < mt; ++i) {
            const float v = fmaf(s, acc[i], out[i]);
            store_c(C + static_cast<int64_t>(m0 + i) * N + n, v, alpha, beta);
        }
    }
}

// Weight-only int8 per output channel: out[m][n] = scale[n] * sum_k A[m][k]*q[k][n].
// The reference composes q8_dequantize_per_col + gemm (src/kernels/quant.cpp:98-105,
// src/kernels/gemm.cpp:21-57).
__global__ void __launch_bounds__(GEN_TN)
gemm_w8a16_generic_kernel(const float* __restrict__ A, const int8_t* __restrict__ Bq,
                          const float* __restrict__ Bs, float* __restrict__ C, int M, int N,
                          int K, float alpha, float beta) {
    __shared__ float As[GEN_TM][GEN_TK];
    const int n = blockIdx.x * GEN_TN + threadIdx.x;
    const int m0 = blockIdx.y * GEN_TM;
    const int mt = min(GEN_TM, M - m0);
    float acc[GEN_TM];
#pragma unroll
    for (int i = 0; i < GEN_TM; ++i) acc[i] = 0.0f;
    for (int k0 = 0; k0 < K; k0 += GEN_TK) {
        const int kt = min(GEN_TK, K - k0);
        __syncthreads();
        for (int i = threadIdx.x; i < GEN_TM * GEN_TK; i += GEN_TN) {
            const int r = i / GEN_TK, c = i % GEN_TK;
            As[r][c] = (r < mt && c < kt) ? A[static_cast<int64_t>(m0 + r) * K + k0 + c] : 0.0f;
        }
        __syncthreads();
        if (n < N) {
            for (int kk = 0; kk < kt; ++kk) {
                const float q = static_cast<float>(Bq[static_cast<int64_t>(k0 + kk) * N + n]);
#pragma unroll
                for (int i = 0; i < GEN_TM; ++i) acc[i] = fmaf(As[i][kk], q, acc[i]);
            }
        }
    }
    if (n < N) {
        const float s = Bs[n];
        for (int i = 0; i < mt; ++i)
            store_c(C + static_cast<int64_t>(m0 + i) * N + n, s * acc[i], alpha, beta);
    }
}

// W8A8: exact int32 dot products, then ((alpha*a_s)*b_s)*float(acc) evaluated
// in the reference's order with single roundings (src/kernels/gemm_quant.cpp:44-46),
// which makes the beta == 0 result bit-identical to the reference.
__device__ __forceinline__ float w8a8_epilogue(float alpha, float a_s, float b_s, int acc) {
    return __fmul_rn(__fmul_rn(__fmul_rn(alpha, a_s), b_s), static_cast<float>(acc));
}

__device__ __forceinline__ void w8a8_store(float* c, float r, float beta) {
    if (beta == 0.0f) *c = r;                       // reference: C = 0, then C += r
    else if (beta == 1.0f) *c = __fadd_rn(*c, r);
    else *c = __fadd_rn(__fmul_rn(*c, beta), r);
}

__global__ void __launch_bounds__(GEN_TN)
gemm_w8a8_generic_kernel(const int8_t* __restrict__ Aq, const int8_t* __restrict__ Bq,
                         const float* __restrict__ a_scales, const float* __restrict__ b_scales,
                         float* __restrict__ C, int M, int N, int K, float alpha, float beta) {
    __shared__ int As[GEN_TM][GEN_TK];
    const int n = blockIdx.x * GEN_TN + threadIdx.x;
    const int m0 = blockIdx.y * GEN_TM;
    const int mt = min(GEN_TM, M - m0);
    int acc[GEN_TM];
#pragma unroll
    for (int i = 0; i < GEN_TM; ++i) acc[i] = 0;
    for (int k0 = 0; k0 < K; k0 += GEN_TK) {
        const int kt = min(GEN_TK, K - k0);
        __syncthreads();
        for (int i = threadIdx.x; i < GEN_TM * GEN_TK; i += GEN_TN) {
            const int r = i / GEN_TK, c = i % GEN_TK;
            As[r][c] = (r < mt && c < kt) ? Aq[static_cast<int64_t>(m0 + r) * K + k0 + c] : 0;
        }
        __syncthreads();
        if (n < N) {
            for (int kk = 0; kk < kt; ++kk) {
                const int q = Bq[static_cast<int64_t>(k0 + kk) * N + n];
#pragma unroll
                for (int i = 0; i < GEN_TM; ++i) acc[i] += As[i][kk] * q;
            }
        }
    }
    if (n < N) {
        const float bs = b_scales[n];
        for (int i = 0; i < mt; ++i)
            w8a8_store(C + static_cast<int64_t>(m0 + i) * N + n,
                       w8a8_epilogue(alpha, a_scales[m0 + i], bs, acc[i]), beta);
    }
}

int launch_w4a16_generic(const float* A, const uint8_t* Bp, const float* Bs, float* C, int M, int N,
                         int K, int G, float alpha, float beta, cudaStream_t st) {
    dim3 grid(ceil_div(N, GEN_TN), ceil_div(M, GEN_TM));
    gemm_w4a16_generic_kernel<<<grid, GEN_TN, 0, st>>>(A, Bp, Bs, C, M, N, K, G, alpha, beta);
    LHB_LAUNCH_CHECK();
    return LHB_OK;
}

int launch_w8a16_generic(const float* A, const int8_t* Bq, const float* Bs, float* C, int M, int N,
                         int K, float alpha, float beta, cudaStream_t st) {
    dim3 grid(ceil_div(N, GEN_TN), ceil_div(M, GEN_TM));
    gemm_w8a16_generic_kernel<<<grid, GEN_TN, 0, st>>>(A, Bq, Bs, C, M, N, K, alpha, beta);
    LHB_LAUNCH_CHECK();
    return LHB_OK;
}

int launch_w8a8_generic(const int8_t* Aq, const int8_t* Bq, const float* as, const float* bs,
                        float* C, int M, int N, int K, float alpha, float beta, cudaStream_t st) {
    dim3 grid(ceil_div(N, GEN_TN), ceil_div(M, GEN_TM));
    gemm_w8a8_generic_kernel<<<grid, GEN_TN, 0, st>>>(Aq, Bq, as, bs, C, M, N, K, alpha, beta);
    LHB_LAUNCH_CHECK();
    return LHB_OK;
}

}  // namespace lhb

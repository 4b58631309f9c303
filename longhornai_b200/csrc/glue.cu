// The element-wise operators between the quantised GEMMs of a decode step:
// RMSNorm (src/kernels/normalization.cpp:58-76), rotary embedding
// (src/kernels/rope.cpp:9-86) and SwiGLU (src/kernels/activation.cpp:12, 46-55).
// The residual adds of a layer need no kernel: they are beta = 1 of the GEMM
// that produces the term.
//
// At decode sizes (rows = requests in flight, a few dozen; dim = 4096..28672)
// these are latency-bound launches of a few hundred KB: one pass over the
// data, 128-bit accesses, no shared-memory staging beyond the block reduction.
// Arithmetic follows the reference's operation order with IEEE intrinsics
// (no FMA contraction), so the only differences from the CPU results are the
// order of the sum of squares and the last-place rounding of the device's
// sinf / cosf / expf.
#include "common.cuh"

namespace lhb {

// One CTA per row.  y = (x * inv_rms) * gamma, inv_rms = 1 / sqrt(sum(x^2) / dim + eps).
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ gamma, float* __restrict__ y,
               int dim, float eps) {
    const int64_t row = blockIdx.x;
    const float* xr = x + row * dim;
    float* yr = y + row * dim;
    __shared__ float red[8];
    const bool vec = (dim & 3) == 0;
    float ss = 0.0f;
    if (vec) {
        for (int i = threadIdx.x * 4; i < dim; i += 1024) {
            const float4 v = *reinterpret_cast<const float4*>(xr + i);
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    } else {
        for (int i = threadIdx.x; i < dim; i += 256) ss += xr[i] * xr[i];
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    ss = red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) ss += red[w];
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, static_cast<float>(dim)), eps)));
    if (vec) {
        for (int i = threadIdx.x * 4; i < dim; i += 1024) {
            const float4 v = *reinterpret_cast<const float4*>(xr + i);      // second read comes from L1/L2
            const float4 g = *reinterpret_cast<const float4*>(gamma + i);
            float4 o;
            o.x = __fmul_rn(__fmul_rn(v.x, inv), g.x);
            o.y = __fmul_rn(__fmul_rn(v.y, inv), g.y);
            o.z = __fmul_rn(__fmul_rn(v.z, inv), g.z);
            o.w = __fmul_rn(__fmul_rn(v.w, inv), g.w);
            *reinterpret_cast<float4*>(yr + i) = o;
        }
    } else {
        for (int i = threadIdx.x; i < dim; i += 256) yr[i] = __fmul_rn(__fmul_rn(xr[i], inv), gamma[i]);
    }
}

// x is [rows, n_heads, head_dim]; row r sits at position pos_offset + r (one
// sequence) or positions[r] + pos_offset (a decode batch: one token per request).
// One thread per (row, head, pair).
__global__ void __launch_bounds__(256)
rope_kernel(float* __restrict__ x, const int32_t* __restrict__ positions, int64_t n_pairs, int n_heads,
            int head_dim, float theta_base, float freq_scale, int interleaved, int pos_offset) {
    const int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (idx >= n_pairs) return;
    const int half = head_dim >> 1;
    const int i = static_cast<int>(idx % half);
    const int64_t rh = idx / half;                       // row * n_heads + head
    const int row = static_cast<int>(rh / n_heads);
    const int p = positions ? positions[row] + pos_offset : pos_offset + row;
    float sn, c;
    rope_sincos(p, i, head_dim, theta_base, freq_scale, &sn, &c);
    float* v = x + rh * head_dim;
    if (interleaved) {
        const float2 ab = *reinterpret_cast<const float2*>(v + 2 * i);
        float2 o;
        o.x = __fsub_rn(__fmul_rn(ab.x, c), __fmul_rn(ab.y, sn));
        o.y = __fadd_rn(__fmul_rn(ab.x, sn), __fmul_rn(ab.y, c));
        *reinterpret_cast<float2*>(v + 2 * i) = o;
    } else {
        const float a = v[i], b = v[i + half];
        v[i] = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, sn));
        v[i + half] = __fadd_rn(__fmul_rn(b, c), __fmul_rn(a, sn));
    }
}

// x is [rows, 2*dim] = gate || value; y[r, i] = (gate * sigmoid(gate)) * value.
__global__ void __launch_bounds__(256)
swiglu_kernel(const float* __restrict__ x, float* __restrict__ y, int64_t total, int dim) {
    const int64_t idx = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) * 4;
    if (idx >= total) return;
    const int64_t r = idx / dim;
    const int i = static_cast<int>(idx - r * dim);
    const float* gate = x + r * 2 * dim + i;
    auto one = [](float g, float v) { return swiglu_one(g, v); };
    if ((dim & 3) == 0) {
        const float4 g = *reinterpret_cast<const float4*>(gate);
        const float4 v = *reinterpret_cast<const float4*>(gate + dim);
        *reinterpret_cast<float4*>(y + idx) = make_float4(one(g.x, v.x), one(g.y, v.y), one(g.z, v.z), one(g.w, v.w));
    } else {
        for (int j = 0; j < 4 && idx + j < total; ++j) {     // a group of four may straddle a row
            const int64_t rj = (idx + j) / dim;
            const int ij = static_cast<int>(idx + j - rj * dim);
            y[idx + j] = one(x[rj * 2 * dim + ij], x[rj * 2 * dim + dim + ij]);
        }
    }
}

}  // namespace lhb

using namespace lhb;

#define REQUIRE(cond, code) \
    do {                    \
        if (!(cond)) return (code); \
    } while (0)

extern "C" {

int lhb_rmsnorm(lhb_ctx* ctx, const float* x, const float* gamma, float* y, int rows, int dim, float eps,
                void* stream) {
    REQUIRE(ctx && x && gamma && y, LHB_ERR_NULL);
    REQUIRE(rows >= 0 && dim > 0, LHB_ERR_BAD_SHAPE);
    if ((dim & 3) == 0)
        REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(gamma) |
                  reinterpret_cast<uintptr_t>(y)) & 15) == 0, LHB_ERR_MISALIGNED);
    if (rows == 0) return LHB_OK;
    rmsnorm_kernel<<<rows, 256, 0, as_stream(stream)>>>(x, gamma, y, dim, eps);
    LHB_LAUNCH_CHECK();
    return LHB_OK;
}

static int launch_rope(float* x, const int32_t* positions, int rows, int n_heads, int head_dim, float theta_base,
                       float freq_scale, int interleaved, int pos_offset, void* stream) {
    REQUIRE(x, LHB_ERR_NULL);
    REQUIRE(rows >= 0 && n_heads > 0 && head_dim > 0 && (head_dim & 1) == 0, LHB_ERR_BAD_SHAPE);
    REQUIRE((reinterpret_cast<uintptr_t>(x) & 7) == 0, LHB_ERR_MISALIGNED);
    const int64_t n_pairs = static_cast<int64_t>(rows) * n_heads * (head_dim / 2);
    if (n_pairs == 0) return LHB_OK;
    rope_kernel<<<static_cast<unsigned>(ceil_div64(n_pairs, 256)), 256, 0, as_stream(stream)>>>(
        x, positions, n_pairs, n_heads, head_dim, theta_base, freq_scale, interleaved, pos_offset);
    LHB_LAUNCH_CHECK();
    return LHB_OK;
}

int lhb_rope(lhb_ctx* ctx, float* x, int seq, int n_heads, int head_dim, float theta_base, float freq_scale,
             int interleaved, int pos_offset, void* stream) {
    REQUIRE(ctx, LHB_ERR_NULL);
    return launch_rope(x, nullptr, seq, n_heads, head_dim, theta_base, freq_scale, interleaved, pos_offset, stream);
}

int lhb_rope_decode_batched(lhb_ctx* ctx, float* x, const int32_t* positions, int n_requests, int n_heads,
                            int head_dim, float theta_base, float freq_scale, int interleaved, void* stream) {
    REQUIRE(ctx && positions, LHB_ERR_NULL);
    return launch_rope(x, positions, n_requests, n_heads, head_dim, theta_base, freq_scale, interleaved, 0, stream);
}

int lhb_swiglu(lhb_ctx* ctx, const float* x, float* y, int rows, int dim, void* stream) {
    REQUIRE(ctx && x && y, LHB_ERR_NULL);
    REQUIRE(rows >= 0 && dim > 0, LHB_ERR_BAD_SHAPE);
    if ((dim & 3) == 0)
        REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0, LHB_ERR_MISALIGNED);
    const int64_t total = static_cast<int64_t>(rows) * dim;
    if (total == 0) return LHB_OK;
    swiglu_kernel<<<static_cast<unsigned>(ceil_div64(ceil_div64(total, 4), 256)), 256, 0, as_stream(stream)>>>(
        x, y, total, dim);
    LHB_LAUNCH_CHECK();
    return LHB_OK;
}

}  // extern "C"

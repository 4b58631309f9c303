// The reference's unit tests for the quantized decode path, re-expressed
// against the GPU drop-in (include/lh_dropin): same shapes, seeds, call
// sequences and acceptance bounds as tests/test_quant.cpp,
// tests/test_gemm_quant.cpp, tests/test_kvcache_quant.cpp and (RMSNorm, RoPE, SwiGLU cases)
// tests/test_normalization.cpp, tests/test_rope.cpp, tests/test_activation.cpp of the reference,
// with all-host buffers, exactly as code written for the reference calls them.
// Own minimal harness (the reference uses GoogleTest).
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <random>
#include <vector>

#include "kernels/gemm_quant.hpp"
#include "kernels/kvcache_quant.hpp"
#include "kernels/paged_attention.hpp"
#include "kernels/quant.hpp"

static int g_fail = 0, g_checks = 0;
#define EXPECT(cond)                                                        \
    do {                                                                    \
        ++g_checks;                                                         \
        if (!(cond)) { ++g_fail; std::printf("FAIL %s:%d: %s\n", __FILE__, __LINE__, #cond); } \
    } while (0)

static std::vector<float> random_vector(int64_t n, uint32_t seed, float lo = -1.0f, float hi = 1.0f) {
    std::mt19937 rng(seed);
    std::uniform_real_distribution<float> dist(lo, hi);
    std::vector<float> v(static_cast<size_t>(n));
    for (auto& x : v) x = dist(rng);
    return v;
}

// fp32 anchor (the reference tests compare against its fp32 gemm)
static void gemm_f32(const float* A, const float* B, float* C, int M, int N, int K, float alpha = 1.0f,
                     float beta = 0.0f) {
    for (int i = 0; i < M; ++i)
        for (int j = 0; j < N; ++j) {
            float acc = 0.0f;
            for (int k = 0; k < K; ++k) acc += A[i * K + k] * B[k * N + j];
            C[i * N + j] = alpha * acc + beta * C[i * N + j];
        }
}

static double rms(const std::vector<float>& a, const std::vector<float>& b) {
    double s = 0;
    for (size_t i = 0; i < a.size(); ++i) { const double d = double(a[i]) - b[i]; s += d * d; }
    return std::sqrt(s / a.size());
}
static double rms(const std::vector<float>& a) {
    double s = 0;
    for (double x : a) s += x * x;
    return std::sqrt(s / a.size());
}

static void quant_round_trips() {
    {   // Q8PerRowFollowsRowScale
        constexpr int rows = 8, dim = 64;
        std::vector<float> x(rows * dim);
        for (int r = 0; r < rows; ++r) {
            const float sc = (r == 0) ? 0.01f : (r == rows - 1 ? 100.0f : 1.0f);
            auto row = random_vector(dim, 4100 + r, -sc, sc);
            for (int i = 0; i < dim; ++i) x[r * dim + i] = row[i];
        }
        std::vector<int8_t> q(x.size());
        std::vector<float> scales(rows), d(x.size());
        lh::q8_quantize_per_row(x.data(), q.data(), scales.data(), rows, dim);
        lh::q8_dequantize_per_row(q.data(), scales.data(), d.data(), rows, dim);
        for (int r = 0; r < rows; ++r)
            for (int i = 0; i < dim; ++i) EXPECT(std::fabs(d[r * dim + i] - x[r * dim + i]) < scales[r] + 1e-6f);
    }
    {   // Q8PerColRoundTrip
        constexpr int rows = 16, cols = 32;
        auto x = random_vector(rows * cols, 4200);
        std::vector<int8_t> q(x.size());
        std::vector<float> scales(cols), d(x.size());
        lh::q8_quantize_per_col(x.data(), q.data(), scales.data(), rows, cols);
        lh::q8_dequantize_per_col(q.data(), scales.data(), d.data(), rows, cols);
        for (int c = 0; c < cols; ++c) {
            EXPECT(scales[c] > 0.0f);
            for (int r = 0; r < rows; ++r) EXPECT(std::fabs(d[r * cols + c] - x[r * cols + c]) < scales[c] + 1e-6f);
        }
    }
    {   // Q4GroupwiseRoundTripBoundedByScale + Q4GetMatchesDequantize
        constexpr int K = 64, N = 16, G = 32;
        auto x = random_vector(K * N, 4300);
        std::vector<uint8_t> packed(K * N / 2);
        std::vector<float> scales((K / G) * N), d(K * N);
        lh::q4_quantize_groupwise(x.data(), packed.data(), scales.data(), K, N, G);
        lh::q4_dequantize_groupwise(packed.data(), scales.data(), d.data(), K, N, G);
        for (int k = 0; k < K; ++k)
            for (int n = 0; n < N; ++n) {
                EXPECT(std::fabs(d[k * N + n] - x[k * N + n]) < scales[(k / G) * N + n] + 1e-6f);
                const int8_t got = lh::q4_get(packed.data(), k, n, N);
                EXPECT(got >= -7 && got <= 7);
                EXPECT(d[k * N + n] == got * scales[(k / G) * N + n]);
            }
    }
}

// tests/test_quant.cpp:10-22 and :100-140 of the reference
static void per_tensor_and_fp8() {
    {   // Q8PerTensorRoundTrip
        auto x = random_vector(1024, 4000, -3.0f, 3.0f);
        std::vector<int8_t> q(x.size());
        float scale = 0.0f;
        lh::q8_quantize_per_tensor(x.data(), q.data(), &scale, x.size());
        std::vector<float> d(x.size());
        lh::q8_dequantize_per_tensor(q.data(), scale, d.data(), x.size());
        EXPECT(scale > 0.0f);
        for (size_t i = 0; i < x.size(); ++i) EXPECT(std::fabs(d[i] - x[i]) < scale + 1e-6f);
    }
    {   // Fp8PerTensorRoundTrip
        auto x = random_vector(1024, 4500, -2.0f, 2.0f);
        std::vector<lh::fp8_e4m3> q(x.size());
        float scale = 0.0f;
        lh::fp8_quantize_per_tensor(x.data(), q.data(), &scale, x.size());
        std::vector<float> d(x.size());
        lh::fp8_dequantize_per_tensor(q.data(), scale, d.data(), x.size());
        for (size_t i = 0; i < x.size(); ++i) EXPECT(std::fabs(d[i] - x[i]) < 0.13f * std::fabs(x[i]) + scale);
        // the host-side conversion of the storage type agrees with what the device dequantised
        for (size_t i = 0; i < x.size(); i += 37) EXPECT(d[i] == q[i].to_float() * scale);
    }
    {   // Fp8PerRowFollowsRowScale
        constexpr int rows = 4, dim = 32;
        std::vector<float> x(rows * dim);
        for (int r = 0; r < rows; ++r) {
            const float mag = (r == 0) ? 0.001f : 50.0f;
            auto row = random_vector(dim, static_cast<uint32_t>(4600 + r), -mag, mag);
            for (int i = 0; i < dim; ++i) x[r * dim + i] = row[i];
        }
        std::vector<lh::fp8_e4m3> q(x.size());
        std::vector<float> scales(rows), d(x.size());
        lh::fp8_quantize_per_row(x.data(), q.data(), scales.data(), rows, dim);
        lh::fp8_dequantize_per_row(q.data(), scales.data(), d.data(), rows, dim);
        for (int r = 0; r < rows; ++r)
            for (int i = 0; i < dim; ++i)
                EXPECT(std::fabs(d[r * dim + i] - x[r * dim + i]) < 0.13f * std::fabs(x[r * dim + i]) + scales[r]);
    }
    {   // per column, same bound
        constexpr int rows = 16, cols = 24;
        auto x = random_vector(rows * cols, 4700, -4.0f, 4.0f);
        std::vector<lh::fp8_e4m3> q(x.size());
        std::vector<float> scales(cols), d(x.size());
        lh::fp8_quantize_per_col(x.data(), q.data(), scales.data(), rows, cols);
        lh::fp8_dequantize_per_col(q.data(), scales.data(), d.data(), rows, cols);
        for (int r = 0; r < rows; ++r)
            for (int c = 0; c < cols; ++c)
                EXPECT(std::fabs(d[r * cols + c] - x[r * cols + c]) < 0.13f * std::fabs(x[r * cols + c]) + scales[c]);
    }
    {   // storage type: conversion round trip of exactly representable values, saturation, NaN code
        EXPECT(lh::fp8_e4m3(1.0f).to_float() == 1.0f && lh::fp8_e4m3(-0.375f).to_float() == -0.375f);
        EXPECT(lh::fp8_e4m3(448.0f).bits == 0x7e && lh::fp8_e4m3(1e9f).bits == 0x7e);
        EXPECT(lh::fp8_e4m3(std::nanf("")).bits == 0x7f && std::isnan(lh::fp8_e4m3::from_bits(0xff).to_float()));
    }
    {   // GemmQuant.Fp8MatchesFp32WithinTolerance (tests/test_gemm_quant.cpp:77-95)
        constexpr int M = 16, N = 32, K = 64;
        auto A = random_vector(M * K, 5200), B = random_vector(K * N, 5201);
        std::vector<float> C_fp32(M * N, 0.0f), C_q(M * N, 0.0f);
        gemm_f32(A.data(), B.data(), C_fp32.data(), M, N, K);
        std::vector<lh::fp8_e4m3> A8(M * K), B8(K * N);
        float a_s = 0.0f, b_s = 0.0f;
        lh::fp8_quantize_per_tensor(A.data(), A8.data(), &a_s, M * K);
        lh::fp8_quantize_per_tensor(B.data(), B8.data(), &b_s, K * N);
        lh::gemm_fp8_e4m3(A8.data(), B8.data(), a_s, b_s, C_q.data(), M, N, K);
        EXPECT(rms(C_q, C_fp32) / rms(C_fp32) < 0.10);
    }
}

static void gemm_quant() {
    {   // W8A8MatchesFp32WithinTolerance
        constexpr int M = 32, N = 48, K = 64;
        auto A = random_vector(M * K, 5000), B = random_vector(K * N, 5001);
        std::vector<float> C_fp32(M * N, 0.0f), C_q(M * N, 0.0f), A_s(M), B_s(N);
        gemm_f32(A.data(), B.data(), C_fp32.data(), M, N, K);
        std::vector<int8_t> Aq(M * K), Bq(K * N);
        lh::q8_quantize_per_row(A.data(), Aq.data(), A_s.data(), M, K);
        lh::q8_quantize_per_col(B.data(), Bq.data(), B_s.data(), K, N);
        lh::gemm_w8a8(Aq.data(), Bq.data(), A_s.data(), B_s.data(), C_q.data(), M, N, K);
        EXPECT(rms(C_q, C_fp32) / rms(C_fp32) < 0.05);
    }
    {   // W4A16MatchesFp32WithinTolerance
        constexpr int M = 16, N = 32, K = 64, G = 32;
        auto A = random_vector(M * K, 5100), B = random_vector(K * N, 5101);
        std::vector<float> C_fp32(M * N, 0.0f), C_q(M * N, 0.0f), B_s((K / G) * N);
        gemm_f32(A.data(), B.data(), C_fp32.data(), M, N, K);
        std::vector<uint8_t> Bp(K * N / 2);
        lh::q4_quantize_groupwise(B.data(), Bp.data(), B_s.data(), K, N, G);
        lh::gemm_w4a16_groupwise(A.data(), Bp.data(), B_s.data(), C_q.data(), M, N, K, G);
        EXPECT(rms(C_q, C_fp32) / rms(C_fp32) < 0.10);
    }
    {   // W8A8RespectsBeta
        constexpr int M = 4, N = 4, K = 4;
        auto A = random_vector(M * K, 5300), B = random_vector(K * N, 5301);
        std::vector<float> C0(M * N, 1.5f), A_s(M), B_s(N);
        auto C_fp32 = C0;
        gemm_f32(A.data(), B.data(), C_fp32.data(), M, N, K, 0.5f, 2.0f);
        std::vector<int8_t> Aq(M * K), Bq(K * N);
        lh::q8_quantize_per_row(A.data(), Aq.data(), A_s.data(), M, K);
        lh::q8_quantize_per_col(B.data(), Bq.data(), B_s.data(), K, N);
        auto C_q = C0;
        lh::gemm_w8a8(Aq.data(), Bq.data(), A_s.data(), B_s.data(), C_q.data(), M, N, K, 0.5f, 2.0f);
        EXPECT(rms(C_q, C_fp32) / rms(C_fp32) < 0.05);
    }
}

static void kv_quant() {
    {   // Q8AppendRoundTripsWithinTolerance
        constexpr int kvh = 2, S = 9, D = 8, bs = 4;
        auto K = random_vector(kvh * S * D, 2200), V = random_vector(kvh * S * D, 2201);
        lh::PagedCacheLayout L;
        L.num_blocks = 4; L.block_size = bs; L.n_kv_heads = kvh; L.head_dim = D;
        const int64_t pool_n = int64_t(L.num_blocks) * kvh * bs * D, scale_n = int64_t(L.num_blocks) * kvh * bs;
        std::vector<int8_t> Kp(pool_n, 0), Vp(pool_n, 0);
        std::vector<float> Ks(scale_n, 0.0f), Vs(scale_n, 0.0f);
        std::vector<int32_t> table = {0, 1, 2};
        lh::paged_kv_append_q8(Kp.data(), Vp.data(), Ks.data(), Vs.data(), K.data(), V.data(), table.data(), L, 0, S);
        for (int h = 0; h < kvh; ++h)
            for (int s = 0; s < S; ++s) {
                const float ks = Ks[lh::paged_scale_offset(L, table[s / bs], h, s % bs)];
                const int64_t off = lh::paged_offset(L, table[s / bs], h, s % bs, 0);
                for (int t = 0; t < D; ++t) EXPECT(std::fabs(Kp[off + t] * ks - K[(h * S + s) * D + t]) < ks + 1e-6f);
            }
    }
    {   // Q8AttentionMatchesFp32WithinTolerance
        constexpr int qh = 4, kvh = 2, sq = 1, sk = 32, d = 16, bs = 8;
        auto Q = random_vector(qh * sq * d, 2300), K = random_vector(kvh * sk * d, 2301),
             V = random_vector(kvh * sk * d, 2302);
        lh::PagedCacheLayout L;
        L.num_blocks = 8; L.block_size = bs; L.n_kv_heads = kvh; L.head_dim = d;
        std::vector<int32_t> table = {0, 1, 2, 3};
        const size_t pn = size_t(L.num_blocks) * kvh * bs * d;
        std::vector<float> Kf(pn, 0.0f), Vf(pn, 0.0f);
        lh::paged_kv_append(Kf.data(), Vf.data(), K.data(), V.data(), table.data(), L, 0, sk);
        lh::PagedAttnConfig cfg;
        cfg.n_q_heads = qh; cfg.n_kv_heads = kvh; cfg.seq_q = sq; cfg.head_dim = d; cfg.causal = true;
        std::vector<float> O_f32(qh * sq * d, 0.0f), O_q8(qh * sq * d, 0.0f);
        lh::paged_attention(Q.data(), Kf.data(), Vf.data(), table.data(), sk, O_f32.data(), cfg, L);
        std::vector<int8_t> Kq(pn, 0), Vq(pn, 0);
        std::vector<float> Ks(pn / d, 0.0f), Vs(pn / d, 0.0f);
        lh::paged_kv_append_q8(Kq.data(), Vq.data(), Ks.data(), Vs.data(), K.data(), V.data(), table.data(), L, 0, sk);
        lh::paged_attention_q8(Q.data(), Kq.data(), Vq.data(), Ks.data(), Vs.data(), table.data(), sk, O_q8.data(),
                               cfg, L);
        double mse = 0;
        for (size_t i = 0; i < O_q8.size(); ++i) {
            mse += (double(O_q8[i]) - O_f32[i]) * (double(O_q8[i]) - O_f32[i]);
            EXPECT(std::fabs(O_q8[i] - O_f32[i]) < 5e-2f);
        }
        EXPECT(mse / O_q8.size() < 1e-3);
        EXPECT(rms(O_f32) > 1e-3);     // the anchor is not trivially zero
    }
}

// RmsNorm.MatchesReference (17 x 96), Rope.* (12x4x64 interleaved, 9x3x48 half rotation with
// scale 0.5 and offset 2, norm preservation on 5x2x32) and Activation.SwiGLU (7 x 32), each
// against the plain loop the reference's *_ref function or test body spells out.
static void decode_glue() {
    {
        const int rows = 17, dim = 96;
        auto x = random_vector(rows * dim, 121, -4.0f, 4.0f);
        auto g = random_vector(dim, 122);
        std::vector<float> y(rows * dim);
        lh::b200::rmsnorm(x.data(), g.data(), y.data(), rows, dim);
        for (int r = 0; r < rows; ++r) {
            float ss = 0.0f;
            for (int i = 0; i < dim; ++i) ss += x[r * dim + i] * x[r * dim + i];
            const float inv = 1.0f / std::sqrt(ss / dim + 1e-5f);
            for (int i = 0; i < dim; ++i)
                EXPECT(std::fabs(y[r * dim + i] - x[r * dim + i] * inv * g[i]) <= 1e-5f + 1e-5f * std::fabs(y[r * dim + i]));
        }
    }
    auto rope_loop = [](std::vector<float>& v, int seq, int n_heads, int hd, float theta, float fs, bool inter, int off) {
        const int half = hd / 2;
        for (int s = 0; s < seq; ++s)
            for (int h = 0; h < n_heads; ++h)
                for (int i = 0; i < half; ++i) {
                    const float ang = static_cast<float>(off + s) * fs * (1.0f / std::pow(theta, static_cast<float>(2 * i) / hd));
                    const float c = std::cos(ang), sn = std::sin(ang);
                    float* p = v.data() + (static_cast<size_t>(s) * n_heads + h) * hd;
                    const int ia = inter ? 2 * i : i, ib = inter ? 2 * i + 1 : i + half;
                    const float a = p[ia], b = p[ib];
                    p[ia] = a * c - b * sn;
                    p[ib] = inter ? a * sn + b * c : b * c + a * sn;
                }
    };
    for (int variant = 0; variant < 2; ++variant) {
        const int seq = variant ? 9 : 12, n_heads = variant ? 3 : 4, hd = variant ? 48 : 64;
        auto base = random_vector(seq * n_heads * hd, 501 + variant);
        auto x = base, want = base;
        lh::b200::rope(x.data(), seq, n_heads, hd, 10000.0f, variant ? 0.5f : 1.0f, variant == 0, variant ? 2 : 0);
        rope_loop(want, seq, n_heads, hd, 10000.0f, variant ? 0.5f : 1.0f, variant == 0, variant ? 2 : 0);
        for (size_t i = 0; i < x.size(); ++i) EXPECT(std::fabs(x[i] - want[i]) <= 1e-5f + 1e-5f * std::fabs(want[i]));
    }
    {
        const int seq = 5, n_heads = 2, hd = 32;
        auto base = random_vector(seq * n_heads * hd, 503);
        auto x = base;
        lh::b200::rope(x.data(), seq, n_heads, hd);
        for (size_t i = 0; i < base.size(); i += 2) {
            const double n0 = base[i] * base[i] + base[i + 1] * base[i + 1];
            const double n1 = x[i] * x[i] + x[i + 1] * x[i + 1];
            EXPECT(std::fabs(n0 - n1) <= 1e-3);
        }
    }
    {
        const int rows = 7, dim = 32;
        auto x = random_vector(rows * 2 * dim, 203, -4.0f, 4.0f);
        std::vector<float> y(rows * dim);
        lh::b200::swiglu(x.data(), y.data(), rows, dim);
        for (int r = 0; r < rows; ++r)
            for (int i = 0; i < dim; ++i) {
                const float gate = x[r * 2 * dim + i], val = x[r * 2 * dim + dim + i];
                EXPECT(std::fabs(y[r * dim + i] - gate / (1.0f + std::exp(-gate)) * val) <= 1e-5f);
            }
    }
}

int main() {
    try {
        quant_round_trips();
        per_tensor_and_fp8();
        gemm_quant();
        kv_quant();
        decode_glue();
    } catch (const std::exception& e) {
        std::printf("EXCEPTION: %s\n", e.what());
        return 2;
    }
    std::printf("%d checks, %d failures\n", g_checks, g_fail);
    return g_fail ? 1 : 0;
}

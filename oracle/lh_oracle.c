/*
 * CPU oracle for the quantized decode hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain single-threaded C, the arithmetic of the
 * reference library's quantized-decode functions so that the CUDA path can
 * be checked bit-for-bit (integer outputs) or within tolerance (fp32
 * outputs).  Nothing in the product links or calls it: only the tests, the
 * smoke check and the benchmark's CPU-baseline leg may load it.
 *
 * Parity is pinned: every function here is compared with the reference's own
 * compiled code (oracle/_ref, built by oracle/Makefile from the reference's
 * sources) on seeded inputs, and with the fixtures in tests/golden/ that the
 * same compiled reference produced.
 *
 * Build flags matter: compile WITHOUT -ffast-math and WITHOUT -march=native
 * (no FMA contraction), the same way the reference is built, so that the
 * float results agree bit-for-bit with the reference.
 *
 * Each function names the reference file:line it follows.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define LHO_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ */
/* 16-bit float conversions (reference: src/kernels/dtypes.hpp:87-105) */
/* ------------------------------------------------------------------ */

/* fp32 -> bf16 bits, round-to-nearest-even, NaN kept quiet.
 * Reference: src/kernels/dtypes.hpp:87-98. */
LHO_API uint16_t lho_f32_to_bf16_bits(float v) {
    uint32_t u;
    memcpy(&u, &v, 4);
    if (((u >> 23) & 0xffu) == 0xffu && (u & 0x7fffffu) != 0u)
        return (uint16_t)((u >> 16) | 0x40u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

/* bf16 bits -> fp32.  Reference: src/kernels/dtypes.hpp:100-105. */
LHO_API float lho_bf16_bits_to_f32(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* In-place round of an fp32 array to bf16 precision (stored back as fp32). */
LHO_API void lho_round_to_bf16(float* x, int64_t n) {
    for (int64_t i = 0; i < n; ++i)
        x[i] = lho_bf16_bits_to_f32(lho_f32_to_bf16_bits(x[i]));
}

/* ------------------------------------------------------------------ */
/* Symmetric integer rounding helpers                                  */
/* ------------------------------------------------------------------ */

/* Saturating round-half-even to [-lim, lim].
 * Reference: src/kernels/quant.cpp:12-19 (int8), :117-124 (int4),
 * src/kernels/kvcache_quant.cpp:14-23. */
static inline int sat_rne(float v, int lim) {
    if (v >= (float)lim) return lim;
    if (v <= (float)-lim) return -lim;
    int r = (int)lrintf(v);
    if (r > lim) r = lim;
    if (r < -lim) r = -lim;
    return r;
}

static inline float absmax_f32(const float* x, int64_t n, int64_t stride) {
    float m = 0.0f;
    for (int64_t i = 0; i < n; ++i) {
        float a = fabsf(x[i * stride]);
        if (a > m) m = a;
    }
    return m;
}

/* ------------------------------------------------------------------ */
/* int8 quantisers                                                     */
/* ------------------------------------------------------------------ */

/* Per-tensor symmetric int8: one scale = max|x|/127 (1 when all zero),
 * q = sat_rne(x * (1/scale)).  Reference: src/kernels/quant.cpp:33-49. */
LHO_API void lho_q8_quantize_per_tensor(const float* src, int8_t* dst, float* scale_out, int64_t n) {
    float m = absmax_f32(src, n, 1);
    float s = (m > 0.0f) ? m / 127.0f : 1.0f;
    float inv = 1.0f / s;
    for (int64_t i = 0; i < n; ++i) dst[i] = (int8_t)sat_rne(src[i] * inv, 127);
    *scale_out = s;
}

/* Reference: src/kernels/quant.cpp:51-54. */
LHO_API void lho_q8_dequantize_per_tensor(const int8_t* src, float scale, float* dst, int64_t n) {
    for (int64_t i = 0; i < n; ++i) dst[i] = src[i] * scale;
}

/* Per-row (per-token) symmetric int8: scale = max|row|/127 (1 when the row
 * is all zero), q = sat_rne(x * (1/scale)) -- note the reciprocal multiply.
 * Reference: src/kernels/quant.cpp:52-63. */
LHO_API void lho_q8_quantize_per_row(const float* src, int8_t* dst,
                                     float* scales, int rows, int dim) {
    for (int r = 0; r < rows; ++r) {
        const float* x = src + (int64_t)r * dim;
        int8_t* q = dst + (int64_t)r * dim;
        float m = absmax_f32(x, dim, 1);
        float s = (m > 0.0f) ? m / 127.0f : 1.0f;
        float inv = 1.0f / s;
        for (int i = 0; i < dim; ++i) q[i] = (int8_t)sat_rne(x[i] * inv, 127);
        scales[r] = s;
    }
}

/* Reference: src/kernels/quant.cpp:65-73. */
LHO_API void lho_q8_dequantize_per_row(const int8_t* src, const float* scales,
                                       float* dst, int rows, int dim) {
    for (int r = 0; r < rows; ++r)
        for (int i = 0; i < dim; ++i)
            dst[(int64_t)r * dim + i] = src[(int64_t)r * dim + i] * scales[r];
}

/* Per-column (per-output-channel) symmetric int8 of a [rows, cols] matrix:
 * scale[c] = max|col c|/127 (1 when zero), q = sat_rne(x / scale[c]) -- a
 * true division here, unlike the per-row quantiser.
 * Reference: src/kernels/quant.cpp:75-96. */
LHO_API void lho_q8_quantize_per_col(const float* src, int8_t* dst,
                                     float* scales, int rows, int cols) {
    for (int c = 0; c < cols; ++c) {
        float m = absmax_f32(src + c, rows, cols);
        scales[c] = (m > 0.0f) ? m / 127.0f : 1.0f;
    }
    for (int r = 0; r < rows; ++r)
        for (int c = 0; c < cols; ++c)
            dst[(int64_t)r * cols + c] =
                (int8_t)sat_rne(src[(int64_t)r * cols + c] / scales[c], 127);
}

/* Reference: src/kernels/quant.cpp:98-105. */
LHO_API void lho_q8_dequantize_per_col(const int8_t* src, const float* scales,
                                       float* dst, int rows, int cols) {
    for (int r = 0; r < rows; ++r)
        for (int c = 0; c < cols; ++c)
            dst[(int64_t)r * cols + c] = src[(int64_t)r * cols + c] * scales[c];
}

/* ------------------------------------------------------------------ */
/* int4 group-wise                                                     */
/* ------------------------------------------------------------------ */

/* Sign-extend the int4 stored for logical row k, column n of a [K, N] weight
 * packed two-per-byte along K (byte (k/2, n); low nibble = even k).
 * Reference: src/kernels/quant.hpp:68-75. */
static inline int q4_at(const uint8_t* packed, int k, int n, int N) {
    uint8_t b = packed[(int64_t)(k >> 1) * N + n];
    int nib = (k & 1) ? (b >> 4) : (b & 0xf);
    return (nib & 8) ? nib - 16 : nib;
}

LHO_API int lho_q4_get(const uint8_t* packed, int k, int n, int N) {
    return q4_at(packed, k, n, N);
}

/* Group-wise symmetric int4 along K: scale[g, n] = max|w[gG..gG+G, n]|/7
 * (1 when zero); q = sat_rne(w / scale) in [-7, 7] (true division); two's
 * complement nibbles, even k in the low nibble.
 * Reference: src/kernels/quant.cpp:128-160. */
LHO_API void lho_q4_quantize_groupwise(const float* src, uint8_t* packed,
                                       float* scales, int K, int N, int G) {
    int groups = K / G;
    for (int g = 0; g < groups; ++g)
        for (int n = 0; n < N; ++n) {
            float m = absmax_f32(src + (int64_t)g * G * N + n, G, N);
            scales[(int64_t)g * N + n] = (m > 0.0f) ? m / 7.0f : 1.0f;
        }
    for (int k = 0; k < K; k += 2)
        for (int n = 0; n < N; ++n) {
            float s0 = scales[(int64_t)(k / G) * N + n];
            float s1 = scales[(int64_t)((k + 1) / G) * N + n];
            int lo = sat_rne(src[(int64_t)k * N + n] / s0, 7);
            int hi = sat_rne(src[(int64_t)(k + 1) * N + n] / s1, 7);
            packed[(int64_t)(k >> 1) * N + n] =
                (uint8_t)((lo & 0xf) | ((hi & 0xf) << 4));
        }
}

/* Reference: src/kernels/quant.cpp:162-171. */
LHO_API void lho_q4_dequantize_groupwise(const uint8_t* packed,
                                         const float* scales, float* dst,
                                         int K, int N, int G) {
    for (int k = 0; k < K; ++k)
        for (int n = 0; n < N; ++n)
            dst[(int64_t)k * N + n] =
                (float)q4_at(packed, k, n, N) * scales[(int64_t)(k / G) * N + n];
}

/* ------------------------------------------------------------------ */
/* GEMMs                                                               */
/* ------------------------------------------------------------------ */

/* C <- beta*C with the reference's special cases (beta==0 stores zeros even
 * over NaN, beta==1 leaves C alone).
 * Reference: src/kernels/gemm_quant.cpp:12-21, src/kernels/gemm.cpp:28-35. */
static void scale_c(float* C, int M, int N, float beta) {
    int64_t n = (int64_t)M * N;
    if (beta == 0.0f) {
        for (int64_t i = 0; i < n; ++i) C[i] = 0.0f;
    } else if (beta != 1.0f) {
        for (int64_t i = 0; i < n; ++i) C[i] *= beta;
    }
}

/* fp32 GEMM C = alpha*A@B + beta*C, row-major, accumulating into C in
 * ascending k for every (i, j) with the term (alpha*A[i,k])*B[k,j].  The
 * reference's 64^3 blocking visits k in the same ascending order for a given
 * (i, j), so the sums are bit-identical.
 * Reference: src/kernels/gemm.cpp:21-57. */
LHO_API void lho_gemm_f32(const float* A, const float* B, float* C, int M,
                          int N, int K, float alpha, float beta) {
    scale_c(C, M, N, beta);
    for (int i = 0; i < M; ++i) {
        float* c = C + (int64_t)i * N;
        for (int k = 0; k < K; ++k) {
            float a = alpha * A[(int64_t)i * K + k];
            const float* b = B + (int64_t)k * N;
            for (int j = 0; j < N; ++j) c[j] += a * b[j];
        }
    }
}

/* W8A8: int8 x int8 -> int32 exact, then C += alpha*a_s[m]*b_s[n]*float(acc)
 * evaluated left to right.  B is [K, N] with N contiguous.  The k loop is
 * interchanged with the j loop here (row-streaming B); int32 sums are exact,
 * so the result is identical to the reference's column walk.
 * Reference: src/kernels/gemm_quant.cpp:29-49. */
LHO_API void lho_gemm_w8a8(const int8_t* Aq, const int8_t* Bq,
                           const float* a_scales, const float* b_scales,
                           float* C, int M, int N, int K, float alpha,
                           float beta) {
    scale_c(C, M, N, beta);
    int32_t* acc = (int32_t*)malloc(sizeof(int32_t) * (size_t)N);
    for (int i = 0; i < M; ++i) {
        memset(acc, 0, sizeof(int32_t) * (size_t)N);
        for (int k = 0; k < K; ++k) {
            int32_t a = Aq[(int64_t)i * K + k];
            const int8_t* b = Bq + (int64_t)k * N;
            for (int j = 0; j < N; ++j) acc[j] += a * (int32_t)b[j];
        }
        float as = a_scales[i];
        float* c = C + (int64_t)i * N;
        for (int j = 0; j < N; ++j)
            c[j] += alpha * as * b_scales[j] * (float)acc[j];
    }
    free(acc);
}

/* W4A16 group-wise: for each K-group, dequantise q*scale into an fp32 panel
 * and accumulate C[i,:] += (alpha*A[i,k]) * panel[k,:] in ascending k.
 * Reference: src/kernels/gemm_quant.cpp:54-82. */
LHO_API void lho_gemm_w4a16_groupwise(const float* A, const uint8_t* Bp,
                                      const float* b_scales, float* C, int M,
                                      int N, int K, int G, float alpha,
                                      float beta) {
    scale_c(C, M, N, beta);
    float* panel = (float*)malloc(sizeof(float) * (size_t)G * (size_t)N);
    for (int k0 = 0; k0 < K; k0 += G) {
        const float* s = b_scales + (int64_t)(k0 / G) * N;
        for (int kk = 0; kk < G; ++kk)
            for (int n = 0; n < N; ++n)
                panel[(int64_t)kk * N + n] =
                    (float)q4_at(Bp, k0 + kk, n, N) * s[n];
        for (int i = 0; i < M; ++i) {
            float* c = C + (int64_t)i * N;
            for (int kk = 0; kk < G; ++kk) {
                float a = alpha * A[(int64_t)i * K + k0 + kk];
                const float* b = panel + (int64_t)kk * N;
                for (int j = 0; j < N; ++j) c[j] += a * b[j];
            }
        }
    }
    free(panel);
}

/* Weight-only int8 per-channel GEMM.  The reference has no single function
 * for it: it is the composition "dequantise per column, then fp32 GEMM".
 * Reference: src/kernels/quant.cpp:98-105 followed by
 * src/kernels/gemm.cpp:21-57. */
LHO_API void lho_gemm_w8a16_perchannel(const float* A, const int8_t* Bq,
                                       const float* b_scales, float* C, int M,
                                       int N, int K, float alpha, float beta) {
    float* Bd = (float*)malloc(sizeof(float) * (size_t)K * (size_t)N);
    lho_q8_dequantize_per_col(Bq, b_scales, Bd, K, N);
    lho_gemm_f32(A, Bd, C, M, N, K, alpha, beta);
    free(Bd);
}

/* ------------------------------------------------------------------ */
/* Paged KV cache                                                      */
/* ------------------------------------------------------------------ */

/* Mirrors PagedCacheLayout (src/kernels/kvcache.hpp:26-31). */
typedef struct {
    int num_blocks;
    int block_size;
    int n_kv_heads;
    int head_dim;
} lho_layout;

/* Mirrors PagedAttnConfig (src/kernels/paged_attention.hpp:28-37); `causal`
 * is an int here (0/1). */
typedef struct {
    int n_q_heads;
    int n_kv_heads;
    int seq_q;
    int head_dim;
    int causal;
    float scale;
    int window;
    int chunk;
} lho_attn_cfg;

/* Element offset of (block, head, slot, 0) in a [num_blocks, heads,
 * block_size, head_dim] pool.  Reference: src/kernels/kvcache.hpp:34-41. */
static inline int64_t row_off(const lho_layout* L, int block, int head,
                              int slot) {
    return (((int64_t)block * L->n_kv_heads + head) * L->block_size + slot) *
           L->head_dim;
}

/* Offset of the per-row scale in [num_blocks, heads, block_size].
 * Reference: src/kernels/kvcache_quant.hpp:31-36. */
static inline int64_t scale_off(const lho_layout* L, int block, int head,
                                int slot) {
    return ((int64_t)block * L->n_kv_heads + head) * L->block_size + slot;
}

/* fp32 append: copy each new (token, head) row into its page slot.  New rows
 * arrive head-major: [n_kv_heads, seq_new, head_dim].
 * Reference: src/kernels/kvcache.cpp:7-32. */
LHO_API void lho_paged_kv_append_f32(float* k_pool, float* v_pool,
                                     const float* k_new, const float* v_new,
                                     const int32_t* table, const lho_layout* L,
                                     int past_len, int seq_new) {
    for (int s = 0; s < seq_new; ++s) {
        int pos = past_len + s;
        int blk = table[pos / L->block_size];
        int slot = pos % L->block_size;
        for (int h = 0; h < L->n_kv_heads; ++h) {
            int64_t d = row_off(L, blk, h, slot);
            int64_t f = ((int64_t)h * seq_new + s) * L->head_dim;
            memcpy(k_pool + d, k_new + f, sizeof(float) * (size_t)L->head_dim);
            memcpy(v_pool + d, v_new + f, sizeof(float) * (size_t)L->head_dim);
        }
    }
}

/* One head_dim row -> int8 + fp32 scale, reciprocal-multiply idiom.
 * Reference: src/kernels/kvcache_quant.cpp:24-35. */
static void q8_row(const float* x, int8_t* q, float* scale, int d) {
    float m = absmax_f32(x, d, 1);
    float s = (m > 0.0f) ? m / 127.0f : 1.0f;
    float inv = 1.0f / s;
    for (int i = 0; i < d; ++i) q[i] = (int8_t)sat_rne(x[i] * inv, 127);
    *scale = s;
}

/* int8 append.  Reference: src/kernels/kvcache_quant.cpp:58-80. */
LHO_API void lho_paged_kv_append_q8(int8_t* k_pool, int8_t* v_pool,
                                    float* k_scales, float* v_scales,
                                    const float* k_new, const float* v_new,
                                    const int32_t* table, const lho_layout* L,
                                    int past_len, int seq_new) {
    for (int s = 0; s < seq_new; ++s) {
        int pos = past_len + s;
        int blk = table[pos / L->block_size];
        int slot = pos % L->block_size;
        for (int h = 0; h < L->n_kv_heads; ++h) {
            int64_t d = row_off(L, blk, h, slot);
            int64_t so = scale_off(L, blk, h, slot);
            int64_t f = ((int64_t)h * seq_new + s) * L->head_dim;
            q8_row(k_new + f, k_pool + d, k_scales + so, L->head_dim);
            q8_row(v_new + f, v_pool + d, v_scales + so, L->head_dim);
        }
    }
}

/* Key j visible to query row i?  Causal aligns the LAST query row with cache
 * position seq_len-1 (shift = seq_len - seq_q); window keeps the trailing
 * `window` keys; chunk keeps keys in the query's chunk.
 * Reference: src/kernels/kvcache_quant.cpp:42-54,
 * src/kernels/paged_attention.cpp:18-30. */
static inline int visible(const lho_attn_cfg* c, int i, int j, int shift) {
    if (c->causal && j > shift + i) return 0;
    if (c->window > 0 && j < shift + i - c->window + 1) return 0;
    if (c->chunk > 0 && (shift + i) / c->chunk != j / c->chunk) return 0;
    return 1;
}

static inline float softmax_scale(const lho_attn_cfg* c) {
    return (c->scale > 0.0f) ? c->scale : 1.0f / sqrtf((float)c->head_dim);
}

/* Shared three-pass attention over a paged pool; `q8` selects int8 pools with
 * per-row scales (dequantised element-by-element as k*ks, v*vs) or fp32
 * pools.  Pass 1 scores + max, pass 2 exp + sum, pass 3 weighted V sum with
 * p = e * (1/sum).  Rows with no visible key produce zeros.
 * Reference: src/kernels/kvcache_quant.cpp:82-161 (int8),
 * src/kernels/paged_attention.cpp:36-108 (fp32). */
static void attend(const float* Q, const void* Kp, const void* Vp,
                   const float* Ks, const float* Vs, const int32_t* table,
                   int seq_len, float* O, const lho_attn_cfg* c,
                   const lho_layout* L, int q8) {
    const float sc = softmax_scale(c);
    const int group = c->n_q_heads / c->n_kv_heads;
    const int d = c->head_dim;
    const int B = L->block_size;
    const int shift = seq_len - c->seq_q;
    float* w = (float*)calloc((size_t)(seq_len > 0 ? seq_len : 1), sizeof(float));

    for (int h = 0; h < c->n_q_heads; ++h) {
        const int kvh = h / group;
        for (int i = 0; i < c->seq_q; ++i) {
            const float* q = Q + ((int64_t)h * c->seq_q + i) * d;
            float* o = O + ((int64_t)h * c->seq_q + i) * d;
            int last = seq_len - 1;
            if (c->causal && shift + i < last) last = shift + i;
            int first = 0;
            if (c->window > 0 && shift + i - c->window + 1 > 0)
                first = shift + i - c->window + 1;
            for (int t = 0; t < d; ++t) o[t] = 0.0f;
            if (last < first) continue;

            float mx = -INFINITY;
            int any = 0;
            for (int j = first; j <= last; ++j) {
                if (!visible(c, i, j, shift)) continue;
                int blk = table[j / B], slot = j % B;
                float dot = 0.0f;
                if (q8) {
                    const int8_t* k = (const int8_t*)Kp + row_off(L, blk, kvh, slot);
                    float ks = Ks[scale_off(L, blk, kvh, slot)];
                    for (int t = 0; t < d; ++t) dot += q[t] * (k[t] * ks);
                } else {
                    const float* k = (const float*)Kp + row_off(L, blk, kvh, slot);
                    for (int t = 0; t < d; ++t) dot += q[t] * k[t];
                }
                dot *= sc;
                w[j] = dot;
                if (dot > mx) mx = dot;
                any = 1;
            }
            if (!any) continue;

            float sum = 0.0f;
            for (int j = first; j <= last; ++j) {
                if (!visible(c, i, j, shift)) continue;
                w[j] = expf(w[j] - mx);
                sum += w[j];
            }
            const float inv = 1.0f / sum;
            for (int j = first; j <= last; ++j) {
                if (!visible(c, i, j, shift)) continue;
                const float p = w[j] * inv;
                int blk = table[j / B], slot = j % B;
                if (q8) {
                    const int8_t* v = (const int8_t*)Vp + row_off(L, blk, kvh, slot);
                    float vs = Vs[scale_off(L, blk, kvh, slot)];
                    for (int t = 0; t < d; ++t) o[t] += p * (v[t] * vs);
                } else {
                    const float* v = (const float*)Vp + row_off(L, blk, kvh, slot);
                    for (int t = 0; t < d; ++t) o[t] += p * v[t];
                }
            }
        }
    }
    free(w);
}

/* Single-request int8 paged attention.
 * Reference: src/kernels/kvcache_quant.cpp:82-161. */
LHO_API void lho_paged_attention_q8(const float* Q, const int8_t* Kp,
                                    const int8_t* Vp, const float* Ks,
                                    const float* Vs, const int32_t* table,
                                    int seq_len, float* O,
                                    const lho_attn_cfg* c, const lho_layout* L) {
    attend(Q, Kp, Vp, Ks, Vs, table, seq_len, O, c, L, 1);
}

/* Single-request fp32 paged attention.
 * Reference: src/kernels/paged_attention.cpp:112-123. */
LHO_API void lho_paged_attention_f32(const float* Q, const float* Kp,
                                     const float* Vp, const int32_t* table,
                                     int seq_len, float* O,
                                     const lho_attn_cfg* c, const lho_layout* L) {
    attend(Q, Kp, Vp, NULL, NULL, table, seq_len, O, c, L, 0);
}

/* Batched calling convention: Q/O [n_req, n_q_heads, seq_q, head_dim], tables
 * [n_req, max_blocks] row-major, seq_lens [n_req].  The reference offers it
 * for fp32 pools only; the int8 form is the same loop over requests.
 * Reference: src/kernels/paged_attention.cpp:125-148. */
LHO_API void lho_paged_attention_q8_batched(
    const float* Q, const int8_t* Kp, const int8_t* Vp, const float* Ks,
    const float* Vs, const int32_t* tables, int max_blocks,
    const int32_t* seq_lens, int n_req, float* O, const lho_attn_cfg* c,
    const lho_layout* L) {
    int64_t per = (int64_t)c->n_q_heads * c->seq_q * c->head_dim;
    for (int r = 0; r < n_req; ++r)
        attend(Q + r * per, Kp, Vp, Ks, Vs, tables + (int64_t)r * max_blocks,
               seq_lens[r], O + r * per, c, L, 1);
}

LHO_API void lho_paged_attention_f32_batched(
    const float* Q, const float* Kp, const float* Vp, const int32_t* tables,
    int max_blocks, const int32_t* seq_lens, int n_req, float* O,
    const lho_attn_cfg* c, const lho_layout* L) {
    int64_t per = (int64_t)c->n_q_heads * c->seq_q * c->head_dim;
    for (int r = 0; r < n_req; ++r)
        attend(Q + r * per, Kp, Vp, NULL, NULL, tables + (int64_t)r * max_blocks,
               seq_lens[r], O + r * per, c, L, 0);
}

/* ------------------------------------------------------------------ */
/* Bench harness: independent calls of the functions above spread over */
/* host threads (the functions themselves stay single-threaded, as in  */
/* the reference).  Compiled with -fopenmp.                            */
/* ---------------------------------------------------------------------------
 * Decode-step glue: RMSNorm, rotary embedding, SwiGLU.
 * ------------------------------------------------------------------------- */

/* src/kernels/normalization.cpp:58-76 (rmsnorm = rmsnorm_ref): sum of squares in
 * index order, inv_rms = 1 / sqrt(sumsq / dim + eps), y = (x * inv_rms) * gamma. */
LHO_API void lho_rmsnorm(const float* x, const float* gamma, float* y, int rows,
                         int dim, float eps) {
    for (int r = 0; r < rows; ++r) {
        const float* xr = x + (int64_t)r * dim;
        float* yr = y + (int64_t)r * dim;
        float sumsq = 0.0f;
        for (int i = 0; i < dim; ++i) sumsq += xr[i] * xr[i];
        const float inv_rms = 1.0f / sqrtf(sumsq / (float)dim + eps);
        for (int i = 0; i < dim; ++i) yr[i] = xr[i] * inv_rms * gamma[i];
    }
}

/* src/kernels/rope.cpp:9-15 and 47-86 (the table-driven `rope`): pair i of a
 * head rotates by angle = (pos_offset + s) * freq_scale / theta_base^(2i/head_dim);
 * interleaved pairs are (2i, 2i+1), half-rotation pairs are (i, i + head_dim/2).
 * x is [seq, n_heads, head_dim], rotated in place. */
LHO_API void lho_rope(float* x, int seq, int n_heads, int head_dim,
                      float theta_base, float freq_scale, int interleaved,
                      int pos_offset) {
    const int half = head_dim / 2;
    for (int s = 0; s < seq; ++s) {
        const float pos = (float)(pos_offset + s) * freq_scale;
        for (int i = 0; i < half; ++i) {
            const float exponent = (float)(2 * i) / (float)head_dim;
            const float inv_freq = 1.0f / powf(theta_base, exponent);
            const float angle = pos * inv_freq;
            const float c = cosf(angle), sn = sinf(angle);
            for (int h = 0; h < n_heads; ++h) {
                float* v = x + ((int64_t)s * n_heads + h) * head_dim;
                if (interleaved) {
                    const float a = v[2 * i], b = v[2 * i + 1];
                    v[2 * i] = a * c - b * sn;
                    v[2 * i + 1] = a * sn + b * c;
                } else {
                    const float a = v[i], b = v[i + half];
                    v[i] = a * c - b * sn;
                    v[i + half] = b * c + a * sn;
                }
            }
        }
    }
}

/* src/kernels/activation.cpp:12 and 46-55: x is [rows, 2*dim] = gate || value,
 * y[r, i] = (gate * sigmoid(gate)) * value with sigmoid(v) = 1 / (1 + exp(-v)). */
LHO_API void lho_swiglu(const float* x, float* y, int rows, int dim) {
    for (int r = 0; r < rows; ++r) {
        const float* gate = x + (int64_t)r * 2 * dim;
        const float* value = gate + dim;
        float* yr = y + (int64_t)r * dim;
        for (int i = 0; i < dim; ++i) {
            const float sg = 1.0f / (1.0f + expf(-gate[i]));
            yr[i] = (gate[i] * sg) * value[i];
        }
    }
}

/* ---------------------------------------------------------------------------
 * Asymmetric int4 with fp16 scale and zero-point per group (an extension: the
 * reference's int4 is symmetric with fp32 scales, src/kernels/quant.hpp:52-57).
 * Same packing as the symmetric form - byte (k/2, n), low nibble = even k - but
 * the nibble is unsigned, u in [0, 15]; parameters are fp16 [K/G, N] each.
 * Parity of these three functions is NOT pinned by the reference (it has no such
 * scheme); only the fp16 conversion is (against lh::half).
 *   range   lo = min(0, min w), hi = max(0, max w) over the group
 *   scale   s = fp16((hi - lo) / 15), 1 if that is 0
 *   zero    z = clamp(rint(-lo / s), 0, 15)
 *   weight  u = clamp(rint(w / s) + z, 0, 15),   w' = (u - z) * s
 * The loop structure follows quant.cpp:128-171 and gemm_quant.cpp:54-82.
 * ------------------------------------------------------------------------- */

/* fp32 -> fp16 bits, round to nearest even, subnormals kept
 * (src/kernels/dtypes.hpp:17-55 computes the same function). */
LHO_API uint16_t lho_f32_to_f16_bits(float v) {
    uint32_t x;
    memcpy(&x, &v, sizeof x);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const int e = (int)((x >> 23) & 0xff);
    uint32_t m = x & 0x7fffffu;
    if (e == 0xff) return (uint16_t)(sign | (m ? 0x7e00u : 0x7c00u));
    int he = e - 127 + 15;
    if (he >= 31) return (uint16_t)(sign | 0x7c00u);
    uint32_t keep, rest, half_ulp;
    if (he <= 0) {
        if (he < -10) return (uint16_t)sign;
        m |= 0x800000u;
        const int sh = 14 - he;                 /* 14 .. 24 */
        keep = m >> sh;
        rest = m & ((1u << sh) - 1u);
        half_ulp = 1u << (sh - 1);
        he = 0;
    } else {
        keep = m >> 13;
        rest = m & 0x1fffu;
        half_ulp = 0x1000u;
    }
    uint32_t h = ((uint32_t)he << 10) + keep;  /* a mantissa carry runs into the exponent */
    if (rest > half_ulp || (rest == half_ulp && (h & 1u))) ++h;
    return (uint16_t)(sign | h);
}

LHO_API float lho_f16_bits_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const int e = (h >> 10) & 0x1f;
    const uint32_t m = h & 0x3ffu;
    float f;
    if (e == 0) {
        f = ldexpf((float)m, -24);             /* zero or subnormal */
    } else if (e == 31) {
        const uint32_t bits = 0x7f800000u | (m << 13);
        memcpy(&f, &bits, sizeof f);
    } else {
        const uint32_t bits = ((uint32_t)(e - 15 + 127) << 23) | (m << 13);
        memcpy(&f, &bits, sizeof f);
    }
    uint32_t b;
    memcpy(&b, &f, sizeof b);
    b |= sign;
    memcpy(&f, &b, sizeof f);
    return f;
}

LHO_API void lho_q4a_quantize_groupwise(const float* src, uint8_t* packed, uint16_t* scales_h,
                                        uint16_t* zeros_h, int K, int N, int G) {
    const int groups = K / G;
    for (int g = 0; g < groups; ++g) {
        for (int n = 0; n < N; ++n) {
            float lo = 0.0f, hi = 0.0f;
            for (int kk = 0; kk < G; ++kk) {
                const float w = src[(int64_t)(g * G + kk) * N + n];
                lo = fminf(lo, w);
                hi = fmaxf(hi, w);
            }
            float s = lho_f16_bits_to_f32(lho_f32_to_f16_bits((hi - lo) / 15.0f));
            if (!(s > 0.0f)) s = 1.0f;
            long z = lrintf(-lo / s);
            z = z < 0 ? 0 : (z > 15 ? 15 : z);
            scales_h[(int64_t)g * N + n] = lho_f32_to_f16_bits(s);
            zeros_h[(int64_t)g * N + n] = lho_f32_to_f16_bits((float)z);
        }
    }
    for (int r = 0; r < K / 2; ++r) {
        for (int n = 0; n < N; ++n) {
            uint8_t byte = 0;
            for (int half = 0; half < 2; ++half) {
                const int k = 2 * r + half, g = k / G;
                const float s = lho_f16_bits_to_f32(scales_h[(int64_t)g * N + n]);
                const long z = (long)lho_f16_bits_to_f32(zeros_h[(int64_t)g * N + n]);
                long u = lrintf(src[(int64_t)k * N + n] / s) + z;
                u = u < 0 ? 0 : (u > 15 ? 15 : u);
                byte |= (uint8_t)(u << (4 * half));
            }
            packed[(int64_t)r * N + n] = byte;
        }
    }
}

static inline int q4a_get(const uint8_t* packed, int k, int n, int N) {
    const uint8_t b = packed[(int64_t)(k >> 1) * N + n];
    return (k & 1) ? (b >> 4) : (b & 0xf);
}

LHO_API void lho_q4a_dequantize_groupwise(const uint8_t* packed, const uint16_t* scales_h,
                                          const uint16_t* zeros_h, float* dst, int K, int N, int G) {
    for (int k = 0; k < K; ++k)
        for (int n = 0; n < N; ++n) {
            const int g = k / G;
            const int z = (int)lho_f16_bits_to_f32(zeros_h[(int64_t)g * N + n]);
            dst[(int64_t)k * N + n] =
                (float)(q4a_get(packed, k, n, N) - z) * lho_f16_bits_to_f32(scales_h[(int64_t)g * N + n]);
        }
}

/* C = beta*C + alpha * A @ dequant(B): group panel first, then fp32 accumulation in k order,
 * a = alpha * A[i, k] folded in before the product (gemm_quant.cpp:60-80). */
LHO_API void lho_gemm_w4a16_asym(const float* A, const uint8_t* Bp, const uint16_t* scales_h,
                                 const uint16_t* zeros_h, float* C, int M, int N, int K, int G,
                                 float alpha, float beta) {
    scale_c(C, M, N, beta);
    float* panel = (float*)malloc(sizeof(float) * (size_t)G * N);
    for (int k0 = 0; k0 < K; k0 += G) {
        const int g = k0 / G;
        for (int kk = 0; kk < G; ++kk)
            for (int n = 0; n < N; ++n) {
                const int z = (int)lho_f16_bits_to_f32(zeros_h[(int64_t)g * N + n]);
                panel[(int64_t)kk * N + n] =
                    (float)(q4a_get(Bp, k0 + kk, n, N) - z) * lho_f16_bits_to_f32(scales_h[(int64_t)g * N + n]);
            }
        for (int i = 0; i < M; ++i) {
            const float* arow = A + (int64_t)i * K + k0;
            float* crow = C + (int64_t)i * N;
            for (int kk = 0; kk < G; ++kk) {
                const float a = alpha * arow[kk];
                const float* brow = panel + (int64_t)kk * N;
                for (int j = 0; j < N; ++j) crow[j] += a * brow[j];
            }
        }
    }
    free(panel);
}

/* ---------------------------------------------------------------------------
 * FP8 E4M3: conversion, quantisers and GEMM.
 * ------------------------------------------------------------------------- */

/* fp32 -> E4M3 bits (1 sign, 4 exponent bits with bias 7, 3 mantissa bits): round to
 * nearest even, saturate at +-448 (0x7e), NaN and infinities become the one NaN code
 * 0x7f, values below half the smallest subnormal (2^-10) flush to signed zero.
 * Reference: src/kernels/dtypes.hpp:111-159. */
LHO_API uint8_t lho_f32_to_e4m3_bits(float v) {
    uint32_t x;
    memcpy(&x, &v, sizeof x);
    const uint32_t sign = (x >> 24) & 0x80u;
    const int e = (int)((x >> 23) & 0xff);
    uint32_t m = x & 0x7fffffu;
    if (e == 0xff) return (uint8_t)(sign | 0x7fu);
    const int ne = e - 127 + 7;
    if (ne > 15 || (ne == 15 && m > 0x600000u)) return (uint8_t)(sign | 0x7eu);
    uint32_t keep, rest, half_ulp, base;
    if (ne >= 1) {
        keep = m >> 20;
        rest = m & 0xfffffu;
        half_ulp = 0x80000u;
        base = (uint32_t)ne << 3;
    } else {
        if (ne < -2) return (uint8_t)sign;
        m |= 0x800000u;
        const int sh = 21 - ne;                 /* 21 .. 23 */
        keep = m >> sh;
        rest = m & ((1u << sh) - 1u);
        half_ulp = 1u << (sh - 1);
        base = 0;
    }
    uint32_t out = base + keep;                 /* a mantissa carry runs into the exponent */
    if (rest > half_ulp || (rest == half_ulp && (out & 1u))) ++out;
    if (out > 0x7eu) out = 0x7eu;
    return (uint8_t)(sign | out);
}

/* Reference: src/kernels/dtypes.hpp:161-196. */
LHO_API float lho_e4m3_bits_to_f32(uint8_t b) {
    const int e = (b >> 3) & 0xf, m = b & 7;
    float mag;
    if (e == 0xf && m == 7) {
        const uint32_t bits = ((b & 0x80u) ? 0x80000000u : 0u) | 0x7fc00000u;
        memcpy(&mag, &bits, sizeof mag);
        return mag;
    }
    mag = (e == 0) ? ldexpf((float)m, -9) : ldexpf((float)(8 + m), e - 10);
    return (b & 0x80u) ? -mag : mag;
}

/* src/kernels/quant.cpp:176-188: one scale = max|x| / 448 (1 if 0), q = e4m3(x * (1/scale)). */
LHO_API void lho_fp8_quantize_per_tensor(const float* src, uint8_t* dst, float* scale_out, int64_t n) {
    float mx = 0.0f;
    for (int64_t i = 0; i < n; ++i) { const float a = fabsf(src[i]); if (a > mx) mx = a; }
    const float scale = (mx > 0.0f) ? mx / 448.0f : 1.0f;
    const float inv = 1.0f / scale;
    for (int64_t i = 0; i < n; ++i) dst[i] = lho_f32_to_e4m3_bits(src[i] * inv);
    *scale_out = scale;
}

/* src/kernels/quant.cpp:195-206: per row, reciprocal-multiply idiom. */
LHO_API void lho_fp8_quantize_per_row(const float* src, uint8_t* dst, float* scales_out, int rows, int dim) {
    for (int r = 0; r < rows; ++r) {
        const float* row = src + (int64_t)r * dim;
        float mx = 0.0f;
        for (int i = 0; i < dim; ++i) { const float a = fabsf(row[i]); if (a > mx) mx = a; }
        const float scale = (mx > 0.0f) ? mx / 448.0f : 1.0f;
        const float inv = 1.0f / scale;
        for (int i = 0; i < dim; ++i) dst[(int64_t)r * dim + i] = lho_f32_to_e4m3_bits(row[i] * inv);
        scales_out[r] = scale;
    }
}

/* src/kernels/quant.cpp:219-238: per column, true-division idiom. */
LHO_API void lho_fp8_quantize_per_col(const float* src, uint8_t* dst, float* scales_out, int rows, int cols) {
    for (int c = 0; c < cols; ++c) scales_out[c] = 0.0f;
    for (int r = 0; r < rows; ++r)
        for (int c = 0; c < cols; ++c) {
            const float a = fabsf(src[(int64_t)r * cols + c]);
            if (a > scales_out[c]) scales_out[c] = a;
        }
    for (int c = 0; c < cols; ++c) scales_out[c] = (scales_out[c] > 0.0f) ? scales_out[c] / 448.0f : 1.0f;
    for (int r = 0; r < rows; ++r)
        for (int c = 0; c < cols; ++c)
            dst[(int64_t)r * cols + c] = lho_f32_to_e4m3_bits(src[(int64_t)r * cols + c] / scales_out[c]);
}

/* src/kernels/quant.cpp:190-193, 208-217, 240-249: q * scale (per tensor: one scale; per row;
 * per column).  `mode` 0 / 1 / 2 selects which, `scales` has 1 / rows / cols entries. */
LHO_API void lho_fp8_dequantize(const uint8_t* src, const float* scales, float* dst, int rows, int cols, int mode) {
    for (int r = 0; r < rows; ++r)
        for (int c = 0; c < cols; ++c) {
            const float s = mode == 0 ? scales[0] : (mode == 1 ? scales[r] : scales[c]);
            dst[(int64_t)r * cols + c] = lho_e4m3_bits_to_f32(src[(int64_t)r * cols + c]) * s;
        }
}

/* src/kernels/gemm_quant.cpp:87-104: C = beta*C + (alpha * A_scale * B_scale) * sum_k a*b, the sum in
 * fp32 in k order for each (i, j). */
LHO_API void lho_gemm_fp8_e4m3(const uint8_t* A, const uint8_t* B, float A_scale, float B_scale, float* C,
                               int M, int N, int K, float alpha, float beta) {
    scale_c(C, M, N, beta);
    const float combined = alpha * A_scale * B_scale;
    float lut[256];
    for (int i = 0; i < 256; ++i) lut[i] = lho_e4m3_bits_to_f32((uint8_t)i);
    for (int i = 0; i < M; ++i)
        for (int j = 0; j < N; ++j) {
            float acc = 0.0f;
            for (int k = 0; k < K; ++k) acc += lut[A[(int64_t)i * K + k]] * lut[B[(int64_t)k * N + j]];
            C[(int64_t)i * N + j] += combined * acc;
        }
}

/* ------------------------------------------------------------------ */

/* N-sharded W4A16: shard s holds a compact [K/2, n_shard] packed slab, its
 * [K/G, n_shard] scales and its own [M, n_shard] output. */
LHO_API void lho_par_gemm_w4a16_shards(const float* A,
                                       const uint8_t* const* Bp,
                                       const float* const* Bs, float* const* C,
                                       int M, int n_shard, int K, int G,
                                       float alpha, float beta, int shards) {
#pragma omp parallel for schedule(dynamic, 1)
    for (int s = 0; s < shards; ++s)
        lho_gemm_w4a16_groupwise(A, Bp[s], Bs[s], C[s], M, n_shard, K, G, alpha,
                                 beta);
}

LHO_API void lho_par_gemm_w8a16_shards(const float* A, const int8_t* const* Bq,
                                       const float* const* Bs, float* const* C,
                                       int M, int n_shard, int K, float alpha,
                                       float beta, int shards) {
#pragma omp parallel for schedule(dynamic, 1)
    for (int s = 0; s < shards; ++s)
        lho_gemm_w8a16_perchannel(A, Bq[s], Bs[s], C[s], M, n_shard, K, alpha,
                                  beta);
}

/* W8A8 over slabs of `slab` rows of M. */
LHO_API void lho_par_gemm_w8a8_mslabs(const int8_t* Aq, const int8_t* Bq,
                                      const float* a_scales,
                                      const float* b_scales, float* C, int M,
                                      int N, int K, float alpha, float beta,
                                      int slab) {
    int n_slabs = (M + slab - 1) / slab;
#pragma omp parallel for schedule(dynamic, 1)
    for (int s = 0; s < n_slabs; ++s) {
        int m0 = s * slab;
        int m = (M - m0 < slab) ? M - m0 : slab;
        lho_gemm_w8a8(Aq + (int64_t)m0 * K, Bq, a_scales + m0, b_scales,
                      C + (int64_t)m0 * N, m, N, K, alpha, beta);
    }
}

/* One request per task. */
LHO_API void lho_par_paged_attention_q8_batched(
    const float* Q, const int8_t* Kp, const int8_t* Vp, const float* Ks,
    const float* Vs, const int32_t* tables, int max_blocks,
    const int32_t* seq_lens, int n_req, float* O, const lho_attn_cfg* c,
    const lho_layout* L) {
    int64_t per = (int64_t)c->n_q_heads * c->seq_q * c->head_dim;
#pragma omp parallel for schedule(dynamic, 1)
    for (int r = 0; r < n_req; ++r)
        lho_paged_attention_q8(Q + r * per, Kp, Vp, Ks, Vs,
                               tables + (int64_t)r * max_blocks, seq_lens[r],
                               O + r * per, c, L);
}

/* Append for many requests: request r appends seq_new[r] rows at past[r];
 * k_new/v_new of request r start at element offset new_off[r]. */
LHO_API void lho_par_paged_kv_append_q8_batched(
    int8_t* k_pool, int8_t* v_pool, float* k_scales, float* v_scales,
    const float* k_new, const float* v_new, const int64_t* new_off,
    const int32_t* tables, int max_blocks, const int32_t* past,
    const int32_t* seq_new, int n_req, const lho_layout* L) {
#pragma omp parallel for schedule(dynamic, 1)
    for (int r = 0; r < n_req; ++r)
        lho_paged_kv_append_q8(k_pool, v_pool, k_scales, v_scales,
                               k_new + new_off[r], v_new + new_off[r],
                               tables + (int64_t)r * max_blocks, L, past[r],
                               seq_new[r]);
}

LHO_API int lho_max_threads(void) {
#ifdef _OPENMP
    extern int omp_get_max_threads(void);
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Thread count of the harness loops above (a launcher may have exported OMP_NUM_THREADS=1). */
LHO_API void lho_set_threads(int n) {
#ifdef _OPENMP
    extern void omp_set_num_threads(int);
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

// C entry points over the reference library's own compiled code.
// TEST INFRASTRUCTURE ONLY: built by oracle/Makefile into oracle/_ref/ from
// the reference's unmodified sources (include path = the reference's src/),
// used to pin the C restatement in lh_oracle.c, to generate tests/golden/,
// and as the CPU baseline of the benchmark.  The product never loads it.
//
// Every `lhr_*` symbol has the same argument list as the `lho_*` symbol of
// lh_oracle.c, so the Python harness can drive either library.
#include <cstdint>
#include <cstring>

#include "kernels/activation.hpp"
#include "kernels/dtypes.hpp"
#include "kernels/gemm.hpp"
#include "kernels/gemm_quant.hpp"
#include "kernels/kvcache.hpp"
#include "kernels/kvcache_quant.hpp"
#include "kernels/normalization.hpp"
#include "kernels/paged_attention.hpp"
#include "kernels/quant.hpp"
#include "kernels/rope.hpp"
#include "runtime/cache_manager.hpp"
#include "runtime/scheduler.hpp"

#ifdef _OPENMP
#include <omp.h>
#endif

#define LHR_API extern "C" __attribute__((visibility("default")))

namespace {

struct CLayout { int num_blocks, block_size, n_kv_heads, head_dim; };
struct CAttn {
    int n_q_heads, n_kv_heads, seq_q, head_dim, causal;
    float scale;
    int window, chunk;
};

lh::PagedCacheLayout to_layout(const CLayout* c) {
    lh::PagedCacheLayout L;
    L.num_blocks = c->num_blocks;
    L.block_size = c->block_size;
    L.n_kv_heads = c->n_kv_heads;
    L.head_dim = c->head_dim;
    return L;
}

lh::PagedAttnConfig to_cfg(const CAttn* c) {
    lh::PagedAttnConfig p;
    p.n_q_heads = c->n_q_heads;
    p.n_kv_heads = c->n_kv_heads;
    p.seq_q = c->seq_q;
    p.head_dim = c->head_dim;
    p.causal = c->causal != 0;
    p.scale = c->scale;
    p.window = c->window;
    p.chunk = c->chunk;
    return p;
}

}  // namespace

LHR_API uint16_t lhr_f32_to_bf16_bits(float v) { return lh::bfloat16(v).bits; }
LHR_API float lhr_bf16_bits_to_f32(uint16_t b) {
    return lh::detail::bf16_bits_to_float(b);
}
// FP8 E4M3 of the reference (src/kernels/dtypes.hpp:111-196, quant.cpp:176-249, gemm_quant.cpp:87-104)
LHR_API uint8_t lhr_f32_to_e4m3_bits(float v) { return lh::detail::float_to_e4m3_bits(v); }
LHR_API float lhr_e4m3_bits_to_f32(uint8_t b) { return lh::detail::e4m3_bits_to_float(b); }
LHR_API void lhr_fp8_quantize_per_tensor(const float* s, uint8_t* d, float* sc, int64_t n) {
    lh::fp8_quantize_per_tensor(s, reinterpret_cast<lh::fp8_e4m3*>(d), sc, n);
}
LHR_API void lhr_fp8_quantize_per_row(const float* s, uint8_t* d, float* sc, int rows, int dim) {
    lh::fp8_quantize_per_row(s, reinterpret_cast<lh::fp8_e4m3*>(d), sc, rows, dim);
}
LHR_API void lhr_fp8_quantize_per_col(const float* s, uint8_t* d, float* sc, int rows, int cols) {
    lh::fp8_quantize_per_col(s, reinterpret_cast<lh::fp8_e4m3*>(d), sc, rows, cols);
}
LHR_API void lhr_fp8_dequantize(const uint8_t* s, const float* sc, float* d, int rows, int cols, int mode) {
    auto* q = reinterpret_cast<const lh::fp8_e4m3*>(s);
    if (mode == 0) lh::fp8_dequantize_per_tensor(q, sc[0], d, static_cast<int64_t>(rows) * cols);
    else if (mode == 1) lh::fp8_dequantize_per_row(q, sc, d, rows, cols);
    else lh::fp8_dequantize_per_col(q, sc, d, rows, cols);
}
LHR_API void lhr_gemm_fp8_e4m3(const uint8_t* A, const uint8_t* B, float as, float bs, float* C, int M, int N, int K,
                               float alpha, float beta) {
    lh::gemm_fp8_e4m3(reinterpret_cast<const lh::fp8_e4m3*>(A), reinterpret_cast<const lh::fp8_e4m3*>(B), as, bs, C,
                      M, N, K, alpha, beta);
}
// fp16 conversion of the reference (src/kernels/dtypes.hpp:17-85), for pinning the restatement
LHR_API uint16_t lhr_f32_to_f16_bits(float v) { return lh::detail::float_to_half_bits(v); }
LHR_API float lhr_f16_bits_to_f32(uint16_t b) { return lh::detail::half_bits_to_float(b); }
LHR_API void lhr_round_to_bf16(float* x, int64_t n) {
    for (int64_t i = 0; i < n; ++i)
        x[i] = static_cast<float>(lh::bfloat16(x[i]));
}

LHR_API void lhr_q8_quantize_per_tensor(const float* s, int8_t* d, float* sc, int64_t n) {
    lh::q8_quantize_per_tensor(s, d, sc, n);
}
LHR_API void lhr_q8_dequantize_per_tensor(const int8_t* s, float sc, float* d, int64_t n) {
    lh::q8_dequantize_per_tensor(s, sc, d, n);
}
LHR_API void lhr_q8_quantize_per_row(const float* s, int8_t* d, float* sc, int rows, int dim) {
    lh::q8_quantize_per_row(s, d, sc, rows, dim);
}
LHR_API void lhr_q8_dequantize_per_row(const int8_t* s, const float* sc, float* d, int rows, int dim) {
    lh::q8_dequantize_per_row(s, sc, d, rows, dim);
}
LHR_API void lhr_q8_quantize_per_col(const float* s, int8_t* d, float* sc, int rows, int cols) {
    lh::q8_quantize_per_col(s, d, sc, rows, cols);
}
LHR_API void lhr_q8_dequantize_per_col(const int8_t* s, const float* sc, float* d, int rows, int cols) {
    lh::q8_dequantize_per_col(s, sc, d, rows, cols);
}
LHR_API int lhr_q4_get(const uint8_t* p, int k, int n, int N) { return lh::q4_get(p, k, n, N); }
LHR_API void lhr_q4_quantize_groupwise(const float* s, uint8_t* p, float* sc, int K, int N, int G) {
    lh::q4_quantize_groupwise(s, p, sc, K, N, G);
}
LHR_API void lhr_q4_dequantize_groupwise(const uint8_t* p, const float* sc, float* d, int K, int N, int G) {
    lh::q4_dequantize_groupwise(p, sc, d, K, N, G);
}

LHR_API void lhr_gemm_f32(const float* A, const float* B, float* C, int M, int N, int K, float alpha, float beta) {
    lh::gemm(A, B, C, M, N, K, alpha, beta);
}
LHR_API void lhr_gemm_w8a8(const int8_t* A, const int8_t* B, const float* as, const float* bs, float* C,
                           int M, int N, int K, float alpha, float beta) {
    lh::gemm_w8a8(A, B, as, bs, C, M, N, K, alpha, beta);
}
LHR_API void lhr_gemm_w4a16_groupwise(const float* A, const uint8_t* Bp, const float* bs, float* C,
                                      int M, int N, int K, int G, float alpha, float beta) {
    lh::gemm_w4a16_groupwise(A, Bp, bs, C, M, N, K, G, alpha, beta);
}
// Weight-only int8: the reference has no fused call; this is its own
// dequantise-then-GEMM composition.
LHR_API void lhr_gemm_w8a16_perchannel(const float* A, const int8_t* Bq, const float* bs, float* C,
                                       int M, int N, int K, float alpha, float beta) {
    float* Bd = new float[static_cast<size_t>(K) * N];
    lh::q8_dequantize_per_col(Bq, bs, Bd, K, N);
    lh::gemm(A, Bd, C, M, N, K, alpha, beta);
    delete[] Bd;
}

LHR_API void lhr_paged_kv_append_f32(float* kp, float* vp, const float* kn, const float* vn,
                                     const int32_t* table, const CLayout* L, int past, int seq_new) {
    lh::paged_kv_append(kp, vp, kn, vn, table, to_layout(L), past, seq_new);
}
LHR_API void lhr_paged_kv_append_q8(int8_t* kp, int8_t* vp, float* ks, float* vs, const float* kn,
                                    const float* vn, const int32_t* table, const CLayout* L,
                                    int past, int seq_new) {
    lh::paged_kv_append_q8(kp, vp, ks, vs, kn, vn, table, to_layout(L), past, seq_new);
}
LHR_API void lhr_paged_attention_q8(const float* Q, const int8_t* kp, const int8_t* vp, const float* ks,
                                    const float* vs, const int32_t* table, int seq_len, float* O,
                                    const CAttn* c, const CLayout* L) {
    lh::paged_attention_q8(Q, kp, vp, ks, vs, table, seq_len, O, to_cfg(c), to_layout(L));
}
LHR_API void lhr_paged_attention_f32(const float* Q, const float* kp, const float* vp,
                                     const int32_t* table, int seq_len, float* O, const CAttn* c,
                                     const CLayout* L) {
    lh::paged_attention(Q, kp, vp, table, seq_len, O, to_cfg(c), to_layout(L));
}
LHR_API void lhr_paged_attention_q8_batched(const float* Q, const int8_t* kp, const int8_t* vp,
                                            const float* ks, const float* vs, const int32_t* tables,
                                            int max_blocks, const int32_t* seq_lens, int n_req,
                                            float* O, const CAttn* c, const CLayout* L) {
    const auto cfg = to_cfg(c);
    const auto lay = to_layout(L);
    const int64_t per = static_cast<int64_t>(cfg.n_q_heads) * cfg.seq_q * cfg.head_dim;
    for (int r = 0; r < n_req; ++r)
        lh::paged_attention_q8(Q + r * per, kp, vp, ks, vs, tables + static_cast<int64_t>(r) * max_blocks,
                               seq_lens[r], O + r * per, cfg, lay);
}
LHR_API void lhr_paged_attention_f32_batched(const float* Q, const float* kp, const float* vp,
                                             const int32_t* tables, int max_blocks,
                                             const int32_t* seq_lens, int n_req, float* O,
                                             const CAttn* c, const CLayout* L) {
    lh::paged_attention_batched(Q, kp, vp, tables, max_blocks, seq_lens, n_req, O, to_cfg(c),
                                to_layout(L));
}

// --- bench harness: independent calls of the unmodified functions spread over
// --- host threads (the reference's kernels contain no parallel region).

LHR_API void lhr_rmsnorm(const float* x, const float* gamma, float* y, int rows, int dim, float eps) {
    lh::rmsnorm(x, gamma, y, rows, dim, eps);
}
LHR_API void lhr_rope(float* x, int seq, int n_heads, int head_dim, float theta_base, float freq_scale,
                      int interleaved, int pos_offset) {
    lh::rope(x, seq, n_heads, head_dim, theta_base, freq_scale, interleaved != 0, pos_offset);
}
LHR_API void lhr_swiglu(const float* x, float* y, int rows, int dim) { lh::swiglu(x, y, rows, dim); }

LHR_API void lhr_par_gemm_w4a16_shards(const float* A, const uint8_t* const* Bp, const float* const* Bs,
                                       float* const* C, int M, int n_shard, int K, int G, float alpha,
                                       float beta, int shards) {
#pragma omp parallel for schedule(dynamic, 1)
    for (int s = 0; s < shards; ++s)
        lh::gemm_w4a16_groupwise(A, Bp[s], Bs[s], C[s], M, n_shard, K, G, alpha, beta);
}
LHR_API void lhr_par_gemm_w8a16_shards(const float* A, const int8_t* const* Bq, const float* const* Bs,
                                       float* const* C, int M, int n_shard, int K, float alpha,
                                       float beta, int shards) {
#pragma omp parallel for schedule(dynamic, 1)
    for (int s = 0; s < shards; ++s)
        lhr_gemm_w8a16_perchannel(A, Bq[s], Bs[s], C[s], M, n_shard, K, alpha, beta);
}
LHR_API void lhr_par_gemm_w8a8_mslabs(const int8_t* Aq, const int8_t* Bq, const float* as,
                                      const float* bs, float* C, int M, int N, int K, float alpha,
                                      float beta, int slab) {
    const int n_slabs = (M + slab - 1) / slab;
#pragma omp parallel for schedule(dynamic, 1)
    for (int s = 0; s < n_slabs; ++s) {
        const int m0 = s * slab;
        const int m = (M - m0 < slab) ? M - m0 : slab;
        lh::gemm_w8a8(Aq + static_cast<int64_t>(m0) * K, Bq, as + m0, bs,
                      C + static_cast<int64_t>(m0) * N, m, N, K, alpha, beta);
    }
}
LHR_API void lhr_par_paged_attention_q8_batched(const float* Q, const int8_t* kp, const int8_t* vp,
                                                const float* ks, const float* vs, const int32_t* tables,
                                                int max_blocks, const int32_t* seq_lens, int n_req,
                                                float* O, const CAttn* c, const CLayout* L) {
    const auto cfg = to_cfg(c);
    const auto lay = to_layout(L);
    const int64_t per = static_cast<int64_t>(cfg.n_q_heads) * cfg.seq_q * cfg.head_dim;
#pragma omp parallel for schedule(dynamic, 1)
    for (int r = 0; r < n_req; ++r)
        lh::paged_attention_q8(Q + r * per, kp, vp, ks, vs, tables + static_cast<int64_t>(r) * max_blocks,
                               seq_lens[r], O + r * per, cfg, lay);
}
LHR_API void lhr_par_paged_kv_append_q8_batched(int8_t* kp, int8_t* vp, float* ks, float* vs,
                                                const float* kn, const float* vn, const int64_t* new_off,
                                                const int32_t* tables, int max_blocks,
                                                const int32_t* past, const int32_t* seq_new, int n_req,
                                                const CLayout* L) {
    const auto lay = to_layout(L);
#pragma omp parallel for schedule(dynamic, 1)
    for (int r = 0; r < n_req; ++r)
        lh::paged_kv_append_q8(kp, vp, ks, vs, kn + new_off[r], vn + new_off[r],
                               tables + static_cast<int64_t>(r) * max_blocks, lay, past[r], seq_new[r]);
}
LHR_API int lhr_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
// Thread count of the harness loops above (a launcher may have exported OMP_NUM_THREADS=1).
LHR_API void lhr_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

// --- the reference cache manager, for pinning the device cache manager's
// --- allocation order (free list pops ascending ids, LIFO on release).
LHR_API void* lhr_cm_create(const CLayout* L) { return new lh::CacheManager(to_layout(L)); }
LHR_API void lhr_cm_destroy(void* m) { delete static_cast<lh::CacheManager*>(m); }
LHR_API int lhr_cm_create_request(void* m) { return static_cast<lh::CacheManager*>(m)->create_request(); }
LHR_API void lhr_cm_release_request(void* m, int id) { static_cast<lh::CacheManager*>(m)->release_request(id); }
LHR_API int lhr_cm_ensure_capacity(void* m, int id, int seq_len) {
    return static_cast<lh::CacheManager*>(m)->ensure_capacity(id, seq_len) ? 1 : 0;
}
LHR_API void lhr_cm_set_seq_len(void* m, int id, int seq_len) {
    static_cast<lh::CacheManager*>(m)->set_seq_len(id, seq_len);
}
LHR_API int lhr_cm_num_free(void* m) { return static_cast<lh::CacheManager*>(m)->num_free_blocks(); }
LHR_API int lhr_cm_refcount(void* m, int b) { return static_cast<lh::CacheManager*>(m)->refcount(b); }
LHR_API int lhr_cm_seq_len(void* m, int id) { return static_cast<lh::CacheManager*>(m)->blocks(id).seq_len; }
LHR_API int lhr_cm_table(void* m, int id, int32_t* out, int cap) {
    const auto& t = static_cast<lh::CacheManager*>(m)->blocks(id).block_table;
    const int n = static_cast<int>(t.size());
    for (int i = 0; i < n && i < cap; ++i) out[i] = t[static_cast<size_t>(i)];
    return n;
}
LHR_API int lhr_cm_reference_block(void* m, int id, int logical, int physical) {
    return static_cast<lh::CacheManager*>(m)->reference_block(id, logical, physical) ? 1 : 0;
}
LHR_API int lhr_cm_allocate_block(void* m) { return static_cast<lh::CacheManager*>(m)->allocate_block(); }
LHR_API void lhr_cm_release_block(void* m, int b) { static_cast<lh::CacheManager*>(m)->release_block(b); }

// --- the reference scheduler, for pinning the device scheduler's lifecycle rules
//     (src/runtime/scheduler.hpp).  Requests are (prompt length, max_new_tokens).
struct RefSched {
    lh::CacheManager* mgr;
    lh::Scheduler* sched;
    lh::ActiveStep last;
};
LHR_API void* lhr_sched_create(void* cm, int max_concurrent) {
    auto* m = static_cast<lh::CacheManager*>(cm);
    return new RefSched{m, new lh::Scheduler(*m, max_concurrent), {}};
}
LHR_API void lhr_sched_destroy(void* s) {
    auto* r = static_cast<RefSched*>(s);
    delete r->sched;
    delete r;
}
LHR_API int lhr_sched_submit(void* s, int prompt_len, int max_new_tokens) {
    lh::Request q;
    q.prompt_tokens.assign(static_cast<size_t>(prompt_len), 0);
    q.max_new_tokens = max_new_tokens;
    return static_cast<RefSched*>(s)->sched->submit(std::move(q));
}
LHR_API int lhr_sched_has_work(void* s) { return static_cast<RefSched*>(s)->sched->has_work() ? 1 : 0; }
LHR_API int lhr_sched_queue_depth(void* s) { return static_cast<int>(static_cast<RefSched*>(s)->sched->queue_depth()); }
LHR_API int lhr_sched_active_size(void* s) { return static_cast<int>(static_cast<RefSched*>(s)->sched->active_size()); }
LHR_API double lhr_sched_last_step_occupancy(void* s) { return static_cast<RefSched*>(s)->sched->last_step_occupancy(); }
LHR_API int lhr_sched_generated(void* s, int id) { return static_cast<RefSched*>(s)->sched->generated(id); }
// prepare_step; returns n_active and keeps the view for the getters below
LHR_API int lhr_sched_prepare_step(void* s) {
    auto* r = static_cast<RefSched*>(s);
    r->last = r->sched->prepare_step();
    return r->last.n_active();
}
LHR_API int lhr_sched_step_max_blocks(void* s) { return static_cast<RefSched*>(s)->last.max_blocks_per_req; }
LHR_API void lhr_sched_step_view(void* s, int32_t* ids, int32_t* seq_lens, int32_t* tables) {
    auto* r = static_cast<RefSched*>(s);
    const auto& v = r->last;
    for (size_t i = 0; i < v.ids.size(); ++i) { ids[i] = v.ids[i]; seq_lens[i] = v.seq_lens[i]; }
    for (size_t i = 0; i < v.block_tables.size(); ++i) tables[i] = v.block_tables[i];
}
LHR_API void lhr_sched_commit_step(void* s, const uint8_t* completed, int n) {
    std::vector<bool> c(static_cast<size_t>(n));
    for (int i = 0; i < n; ++i) c[i] = completed[i] != 0;
    static_cast<RefSched*>(s)->sched->commit_step(c, std::vector<int32_t>(static_cast<size_t>(n), 0));
}


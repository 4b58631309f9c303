// C ABI: context management, argument validation and dispatch between the
// tensor-core fast paths and the generic kernels.  The quantiser and append
// entry points live next to their kernels (quant.cu, kvcache.cu).
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "common.cuh"
#include "dispatch.h"

namespace lhb {

static thread_local std::string g_last_error;

void set_last_error(const char* what, cudaError_t err) {
    g_last_error = std::string(what) + ": " + cudaGetErrorName(err) + " (" + cudaGetErrorString(err) + ")";
    // leave the runtime's sticky "last error" cleared for non-fatal errors
    cudaGetLastError();
}
void set_last_error_text(const std::string& text) { g_last_error = text; }

}  // namespace lhb

using namespace lhb;

extern "C" {

const char* lhb_last_error(void) { return g_last_error.c_str(); }

const char* lhb_status_string(int s) {
    switch (s) {
        case LHB_OK: return "ok";
        case LHB_ERR_BAD_SHAPE: return "bad shape";
        case LHB_ERR_MISALIGNED: return "pointer not 16-byte aligned";
        case LHB_ERR_UNSUPPORTED: return "unsupported configuration";
        case LHB_ERR_CUDA: return "CUDA error";
        case LHB_ERR_NULL: return "null pointer";
        case LHB_ERR_SCRATCH: return "scratch arena too small";
        case LHB_ERR_TIMEOUT: return "device-side wait timed out";
        default: return "unknown status";
    }
}

int lhb_ctx_create(int device, size_t scratch_bytes, lhb_ctx** out) {
    if (!out) return LHB_ERR_NULL;
    *out = nullptr;
    int n_dev = 0;
    LHB_CUDA(cudaGetDeviceCount(&n_dev));
    if (device < 0 || device >= n_dev) return LHB_ERR_BAD_SHAPE;
    LHB_CUDA(cudaSetDevice(device));
    lhb_ctx* c = new lhb_ctx();
    c->device = device;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) { delete c; return LHB_ERR_CUDA; }
    c->sm_count = prop.multiProcessorCount;
    c->scratch_bytes = scratch_bytes ? scratch_bytes : (size_t(64) << 20);
    c->counters_len = 1 << 16;
    if (cudaMalloc(&c->scratch, c->scratch_bytes) != cudaSuccess ||
        cudaMalloc(&c->status_word, sizeof(int)) != cudaSuccess ||
        cudaMalloc(&c->counters, c->counters_len * sizeof(int)) != cudaSuccess) {
        set_last_error("cudaMalloc(context)", cudaGetLastError());
        lhb_ctx_destroy(c);
        return LHB_ERR_CUDA;
    }
    cudaMemset(c->status_word, 0, sizeof(int));
    cudaMemset(c->counters, 0, c->counters_len * sizeof(int));
    cudaDeviceSynchronize();
    *out = c;
    return LHB_OK;
}

int lhb_ctx_destroy(lhb_ctx* c) {
    if (!c) return LHB_ERR_NULL;
    cudaSetDevice(c->device);
    if (c->scratch) cudaFree(c->scratch);
    if (c->status_word) cudaFree(c->status_word);
    if (c->counters) cudaFree(c->counters);
    delete c;
    return LHB_OK;
}

int lhb_ctx_poll(lhb_ctx* c, void* stream) {
    if (!c) return LHB_ERR_NULL;
    int v = 0;
    LHB_CUDA(cudaStreamSynchronize(as_stream(stream)));
    LHB_CUDA(cudaMemcpy(&v, c->status_word, sizeof(int), cudaMemcpyDeviceToHost));
    if (v != 0) {
        // A wait that ran out may have left a split-K or split-KV arrival count short of its
        // reset: zero the counters too, so that the context is usable again after the report.
        LHB_CUDA(cudaMemset(c->status_word, 0, sizeof(int)));
        LHB_CUDA(cudaMemset(c->counters, 0, c->counters_len * sizeof(int)));
    }
    return v;
}

// ---- fast-path predicates -------------------------------------------------

int lhb_gemm_w4a16_fast_path(int M, int N, int K, int G) { return w4a16_fast_ok(M, N, K, G) ? 1 : 0; }
int lhb_gemm_w8a16_fast_path(int M, int N, int K) { return w8a16_fast_ok(M, N, K) ? 1 : 0; }
int lhb_gemm_w8a8_fast_path(int M, int N, int K) { return w8a8_fast_ok(M, N, K) ? 1 : 0; }
int lhb_paged_attention_q8_fast_path(const lhb_paged_attn_cfg* cfg, const lhb_paged_layout* L) {
    return (cfg && L && decode_fast_ok(*cfg, *L)) ? 1 : 0;
}

// ---- GEMMs -------------------------------------------------------------------

int lhb_gemm_w4a16_groupwise(lhb_ctx* ctx, const float* A, const uint8_t* Bp, const float* Bs,
                             float* C, int M, int N, int K, int G, float alpha, float beta,
                             void* stream) {
    if (!ctx || !A || !Bp || !Bs || !C) return LHB_ERR_NULL;
    if (M < 0 || N <= 0 || K <= 0 || G <= 0) return LHB_ERR_BAD_SHAPE;
    if ((K & 1) || (K % G) != 0) return LHB_ERR_BAD_SHAPE;
    if (M == 0) return LHB_OK;
    cudaStream_t st = as_stream(stream);
    const bool al = aligned16(A) && aligned16(Bp) && aligned16(Bs) && aligned16(C);
    if (al && M >= w4a16_tc_min_rows() && w4a16_tc_ok(M, N, K, G))
        return launch_w4a16_tc(ctx, A, Bp, Bs, C, M, N, K, G, alpha, beta, st, 0, nullptr, 0.0f);
    if (w4a16_fast_ok(M, N, K, G) && al)
        return launch_w4a16_fast(ctx, A, Bp, Bs, C, M, N, K, G, alpha, beta, st);
    return launch_w4a16_generic(A, Bp, Bs, C, M, N, K, G, alpha, beta, st);
}

int lhb_gemm_w4a16_groupwise_peer(lhb_ctx* ctx, const float* A, const uint8_t* Bp, const float* Bs, float* C, int M,
                                  int N, int K, int G, float alpha, float beta, void* const* dst_table,
                                  uint32_t* const* flag_table, uint32_t* state, int rank, int world, int timeout_ms,
                                  void* stream) {
    if (!ctx || !A || !Bp || !Bs || !C || !dst_table || !flag_table || !state) return LHB_ERR_NULL;
    if (M <= 0 || N <= 0 || K <= 0 || G <= 0 || (K & 1) || (K % G) != 0) return LHB_ERR_BAD_SHAPE;
    if (world < 1 || world > 64 || rank < 0 || rank >= world || timeout_ms <= 0) return LHB_ERR_BAD_SHAPE;
    if (static_cast<int64_t>(M) * N * world >= (int64_t(1) << 31)) return LHB_ERR_BAD_SHAPE;
    // only the tensor-core kernel pushes its results itself; other shapes: plain GEMM + lhb_peer_allgather_cols
    if (!(M >= w4a16_tc_min_rows() && w4a16_tc_ok(M, N, K, G) && aligned16(A) && aligned16(Bp) && aligned16(Bs) &&
          aligned16(C)))
        return LHB_ERR_UNSUPPORTED;
    cudaStream_t st = as_stream(stream);
    const W4Peer peer{dst_table, flag_table, world, rank, N * world, rank * N};
    uint32_t arrivals = 0;
    const int e = launch_w4a16_tc(ctx, A, Bp, Bs, C, M, N, K, G, alpha, beta, st, 0, nullptr, 0.0f, &peer, &arrivals);
    if (e != LHB_OK && arrivals == 0) return e;              // nothing that signals was launched
    // A failure after some slabs were launched: their tiles still raise every rank's counters, so the wait for
    // exactly those arrivals is issued all the same - the ranks' expected counts stay in step - and the error
    // is what the caller gets.
    const int w = launch_peer_wait(flag_table, state, rank, world, arrivals, timeout_ms, st);
    return e != LHB_OK ? e : w;
}

int lhb_gemm_w8a16_perchannel(lhb_ctx* ctx, const float* A, const int8_t* Bq, const float* Bs,
                              float* C, int M, int N, int K, float alpha, float beta,
                              void* stream) {
    if (!ctx || !A || !Bq || !Bs || !C) return LHB_ERR_NULL;
    if (M < 0 || N <= 0 || K <= 0) return LHB_ERR_BAD_SHAPE;
    if (M == 0) return LHB_OK;
    cudaStream_t st = as_stream(stream);
    if (w8a16_fast_ok(M, N, K) && aligned16(A) && aligned16(Bq) && aligned16(Bs) && aligned16(C))
        return launch_w8a16_fast(ctx, A, Bq, Bs, C, M, N, K, alpha, beta, st);
    return launch_w8a16_generic(A, Bq, Bs, C, M, N, K, alpha, beta, st);
}

int lhb_gemm_w4a16_groupwise_prologue(lhb_ctx* ctx, const float* X, int prologue, const float* gamma, float eps,
                                      const uint8_t* Bp, const float* Bs, float* C, int M, int N, int K, int G,
                                      float alpha, float beta, void* stream) {
    if (!ctx || !X || !Bp || !Bs || !C) return LHB_ERR_NULL;
    if (prologue != 1 && prologue != 2) return LHB_ERR_BAD_SHAPE;
    if (prologue == 1 && !gamma) return LHB_ERR_NULL;
    if (M < 0 || N <= 0 || K <= 0 || G <= 0 || (K % 2) || (K % G)) return LHB_ERR_BAD_SHAPE;
    if (M == 0) return LHB_OK;
    if (M >= w4a16_tc_min_rows() && w4a16_tc_ok(M, N, K, G) && aligned16(X) && aligned16(Bp) && aligned16(Bs) &&
        aligned16(C) && (prologue != 1 || aligned16(gamma)))
        return launch_w4a16_tc(ctx, X, Bp, Bs, C, M, N, K, G, alpha, beta, as_stream(stream), prologue, gamma, eps);
    if (M - ((M - 1) / 16) * 16 <= 2) return LHB_ERR_UNSUPPORTED;   // a last slab of one or two rows has no digit pass
    if (!(w4a16_fast_ok(M, N, K, G) && aligned16(X) && aligned16(Bp) && aligned16(Bs) && aligned16(C) &&
          (prologue != 1 || aligned16(gamma))))
        return LHB_ERR_UNSUPPORTED;       // the caller runs lhb_rmsnorm / lhb_swiglu and the plain GEMM instead
    return launch_w4a16_fast_prologue(ctx, X, prologue, gamma, eps, Bp, Bs, C, M, N, K, G, alpha, beta,
                                      as_stream(stream));
}

int lhb_gemm_w8a8(lhb_ctx* ctx, const int8_t* Aq, const int8_t* Bq, const float* as,
                  const float* bs, float* C, int M, int N, int K, float alpha, float beta,
                  void* stream) {
    if (!ctx || !Aq || !Bq || !as || !bs || !C) return LHB_ERR_NULL;
    if (M < 0 || N <= 0 || K <= 0) return LHB_ERR_BAD_SHAPE;
    if (M == 0) return LHB_OK;
    cudaStream_t st = as_stream(stream);
    if (w8a8_fast_ok(M, N, K) && aligned16(Aq) && aligned16(Bq) && aligned16(bs) && aligned16(C))
        return launch_w8a8_fast(ctx, Aq, Bq, as, bs, C, M, N, K, alpha, beta, st);
    return launch_w8a8_generic(Aq, Bq, as, bs, C, M, N, K, alpha, beta, st);
}

int lhb_gemm_w8a8_sharded(lhb_ctx* ctx, const int8_t* Aq, const int8_t* Bq, const float* as, const float* bs,
                          void* const* full_C, int rank, int world, int M, int N_local, int K, float alpha,
                          void* stream) {
    if (!ctx || !Aq || !Bq || !as || !bs || !full_C) return LHB_ERR_NULL;
    if (M <= 0 || N_local <= 0 || K <= 0) return LHB_ERR_BAD_SHAPE;
    if (world < 1 || world > 8 || rank < 0 || rank >= world) return LHB_ERR_BAD_SHAPE;
    if (static_cast<int64_t>(N_local) * world >= (int64_t(1) << 31)) return LHB_ERR_BAD_SHAPE;
    for (int r = 0; r < world; ++r)
        if (!full_C[r]) return LHB_ERR_NULL;
    // only the tensor-core kernel pushes its tiles itself
    if (!(w8a8_fast_ok(M, N_local, K) && aligned16(Aq) && aligned16(Bq) && aligned16(bs) && (N_local % 32) == 0))   // whole 32-column chunks reach the peers
        return LHB_ERR_UNSUPPORTED;
    float* dst[8];
    dst[0] = static_cast<float*>(full_C[rank]);              // this rank's own copy first (p.C)
    int n = 1;
    for (int d = 1; d < world; ++d) dst[n++] = static_cast<float*>(full_C[(rank + d) % world]);
    for (int d = 0; d < n; ++d)
        if (!aligned16(dst[d])) return LHB_ERR_MISALIGNED;
    return launch_w8a8_sharded(ctx, Aq, Bq, as, bs, dst, n, M, N_local, K, static_cast<int64_t>(N_local) * world,
                               rank * N_local, alpha, as_stream(stream));
}

int lhb_ctx_set_sm_limit(lhb_ctx* ctx, int sm_limit) {
    if (!ctx) return LHB_ERR_NULL;
    if (sm_limit < 0) return LHB_ERR_BAD_SHAPE;
    ctx->sm_limit = sm_limit;
    return LHB_OK;
}

// ---- paged attention ------------------------------------------------------------

static int check_attn(const lhb_paged_attn_cfg* cfg, const lhb_paged_layout* L) {
    if (!cfg || !L) return LHB_ERR_NULL;
    if (L->num_blocks <= 0 || L->block_size <= 0 || L->n_kv_heads <= 0 || L->head_dim <= 0)
        return LHB_ERR_BAD_SHAPE;
    if (cfg->n_q_heads <= 0 || cfg->n_kv_heads <= 0 || cfg->seq_q <= 0 || cfg->head_dim <= 0)
        return LHB_ERR_BAD_SHAPE;
    if (cfg->n_q_heads % cfg->n_kv_heads) return LHB_ERR_BAD_SHAPE;
    if (cfg->head_dim != L->head_dim || cfg->n_kv_heads != L->n_kv_heads) return LHB_ERR_BAD_SHAPE;
    if (cfg->window < 0 || cfg->chunk < 0) return LHB_ERR_BAD_SHAPE;
    if (cfg->seq_q > 65535 || cfg->n_q_heads > 65535) return LHB_ERR_UNSUPPORTED;
    return LHB_OK;
}

int lhb_paged_attention_q8_batched(lhb_ctx* ctx, const float* Q, const int8_t* Kp, const int8_t* Vp,
                                   const float* Ks, const float* Vs, const int32_t* tables,
                                   int max_blocks, const int32_t* seq_lens, int n_req, float* O,
                                   const lhb_paged_attn_cfg* cfg, const lhb_paged_layout* L,
                                   void* stream) {
    if (!ctx || !Q || !Kp || !Vp || !Ks || !Vs || !tables || !seq_lens || !O) return LHB_ERR_NULL;
    if (int e = check_attn(cfg, L)) return e;
    if (n_req < 0 || max_blocks <= 0 || n_req > 65535) return LHB_ERR_BAD_SHAPE;
    if (n_req == 0) return LHB_OK;
    cudaStream_t st = as_stream(stream);
    if (decode_fast_ok(*cfg, *L) && aligned16(Q) && aligned16(Kp) && aligned16(Vp) &&
        aligned16(Ks) && aligned16(Vs) && aligned16(O)) {
        const int e = launch_decode_fast(ctx, Q, Kp, Vp, Ks, Vs, tables, max_blocks, seq_lens, n_req,
                                         O, *cfg, *L, st);
        if (e != LHB_ERR_SCRATCH) return e;
    }
    return launch_paged_attention_generic(ctx, true, Q, Kp, Vp, Ks, Vs, tables, max_blocks, seq_lens,
                                          0, n_req, O, *cfg, *L, st);
}

int lhb_paged_attention_q8(lhb_ctx* ctx, const float* Q, const int8_t* Kp, const int8_t* Vp,
                           const float* Ks, const float* Vs, const int32_t* table, int seq_len,
                           float* O, const lhb_paged_attn_cfg* cfg, const lhb_paged_layout* L,
                           void* stream) {
    if (!ctx || !Q || !Kp || !Vp || !Ks || !Vs || !table || !O) return LHB_ERR_NULL;
    if (int e = check_attn(cfg, L)) return e;
    if (seq_len < 0) return LHB_ERR_BAD_SHAPE;
    // the single-request form knows seq_len on the host; the table length it
    // implies is ceil(seq_len / block_size)
    const int max_blocks = std::max(1, ceil_div(seq_len, L->block_size));
    return launch_paged_attention_generic(ctx, true, Q, Kp, Vp, Ks, Vs, table, max_blocks, nullptr,
                                          seq_len, 1, O, *cfg, *L, as_stream(stream));
}

int lhb_paged_attention_f32_batched(lhb_ctx* ctx, const float* Q, const float* Kp, const float* Vp,
                                    const int32_t* tables, int max_blocks, const int32_t* seq_lens,
                                    int n_req, float* O, const lhb_paged_attn_cfg* cfg,
                                    const lhb_paged_layout* L, void* stream) {
    if (!ctx || !Q || !Kp || !Vp || !tables || !seq_lens || !O) return LHB_ERR_NULL;
    if (int e = check_attn(cfg, L)) return e;
    if (n_req < 0 || max_blocks <= 0 || n_req > 65535) return LHB_ERR_BAD_SHAPE;
    if (n_req == 0) return LHB_OK;
    return launch_paged_attention_generic(ctx, false, Q, Kp, Vp, nullptr, nullptr, tables, max_blocks,
                                          seq_lens, 0, n_req, O, *cfg, *L, as_stream(stream));
}

}  // extern "C"

// The reference's `namespace lh` entry points for the quantized decode path,
// implemented over the C ABI (see include/lh_dropin/lh_dropin.hpp).  Host
// pointers are staged through device memory; device pointers pass through.
#include <algorithm>
#include <cstdio>
#include <mutex>
#include <stdexcept>
#include <string>

#include "common.cuh"
#include "lh_dropin/lh_dropin.hpp"

namespace {

cudaStream_t g_stream = nullptr;

lhb_ctx* context() {
    static std::mutex mu;
    static lhb_ctx* ctxs[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess)
        throw std::runtime_error("lh drop-in: no CUDA device (there is no CPU fallback)");
    std::lock_guard<std::mutex> lk(mu);
    if (!ctxs[dev & 63]) {
        const int e = lhb_ctx_create(dev, 0, &ctxs[dev & 63]);
        if (e) throw std::runtime_error(std::string("lh drop-in: lhb_ctx_create: ") + lhb_status_string(e) +
                                        " " + lhb_last_error());
    }
    return ctxs[dev & 63];
}

void check(int status, const char* where) {
    if (status != LHB_OK)
        throw std::runtime_error(std::string("lh::") + where + ": " + lhb_status_string(status) + " " +
                                 lhb_last_error());
}

void cuda_ok(cudaError_t e, const char* where) {
    if (e != cudaSuccess) throw std::runtime_error(std::string("lh drop-in: ") + where + ": " + cudaGetErrorString(e));
}

bool on_device(const void* p) {
    cudaPointerAttributes a{};
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return false; }
    return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

// One argument of a call: a device view of `n` elements of T that live either
// on the device already or in host memory (then staged).
template <class T>
class Arg {
public:
    enum Mode { In, Out, InOut };
    Arg(const T* p, size_t n, Mode mode, bool& any_host) : host_(const_cast<T*>(p)), n_(n), mode_(mode) {
        if (n == 0 || p == nullptr || on_device(p)) { dev_ = const_cast<T*>(p); return; }
        any_host = true;
        staged_ = true;
        cuda_ok(cudaMalloc(&dev_, n * sizeof(T)), "cudaMalloc(staging)");
        if (mode != Out)
            cuda_ok(cudaMemcpyAsync(dev_, p, n * sizeof(T), cudaMemcpyHostToDevice, g_stream), "H2D");
    }
    ~Arg() { if (staged_) cudaFree(dev_); }
    Arg(const Arg&) = delete;
    T* get() const { return dev_; }
    void writeback() {
        if (staged_ && mode_ != In)
            cuda_ok(cudaMemcpyAsync(host_, dev_, n_ * sizeof(T), cudaMemcpyDeviceToHost, g_stream), "D2H");
    }
private:
    T* host_;
    T* dev_ = nullptr;
    size_t n_;
    Mode mode_;
    bool staged_ = false;
};

void finish(bool any_host) {
    if (any_host) cuda_ok(cudaStreamSynchronize(g_stream), "synchronize");
}

lhb_paged_layout to_c(const lh::PagedCacheLayout& L) { return {L.num_blocks, L.block_size, L.n_kv_heads, L.head_dim}; }
lhb_paged_attn_cfg to_c(const lh::PagedAttnConfig& c) {
    return {c.n_q_heads, c.n_kv_heads, c.seq_q, c.head_dim, c.causal ? 1 : 0, c.scale, c.window, c.chunk};
}
size_t pool_elems(const lh::PagedCacheLayout& L) {
    return static_cast<size_t>(L.num_blocks) * L.n_kv_heads * L.block_size * L.head_dim;
}
size_t scale_elems(const lh::PagedCacheLayout& L) {
    return static_cast<size_t>(L.num_blocks) * L.n_kv_heads * L.block_size;
}
size_t sz(int64_t a, int64_t b = 1, int64_t c = 1) { return static_cast<size_t>(a * b * c); }

}  // namespace

namespace lh {

namespace dropin {
void set_stream(void* s) { g_stream = static_cast<cudaStream_t>(s); }
void* stream() { return g_stream; }
void synchronize() { cuda_ok(cudaStreamSynchronize(g_stream), "synchronize"); }
}  // namespace dropin

#define ARG(T, name, ptr, n, mode) Arg<T> name(ptr, n, Arg<T>::mode, any_host)

void q8_quantize_per_tensor(const float* src, int8_t* dst, float* scale_out, int64_t n) {
    bool any_host = false;
    ARG(float, s, src, sz(n), In); ARG(int8_t, d, dst, sz(n), Out); ARG(float, sc, scale_out, 1, Out);
    check(lhb_q8_quantize_per_tensor(context(), s.get(), d.get(), sc.get(), n, g_stream), "q8_quantize_per_tensor");
    d.writeback(); sc.writeback(); finish(any_host);
}

void q8_dequantize_per_tensor(const int8_t* src, float scale, float* dst, int64_t n) {
    bool any_host = false;
    ARG(int8_t, s, src, sz(n), In); ARG(float, d, dst, sz(n), Out);
    check(lhb_q8_dequantize_per_tensor(context(), s.get(), scale, d.get(), n, g_stream), "q8_dequantize_per_tensor");
    d.writeback(); finish(any_host);
}

// E4M3 buffers are byte buffers of the storage codes
static const uint8_t* bytes(const fp8_e4m3* p) { return reinterpret_cast<const uint8_t*>(p); }
static uint8_t* bytes(fp8_e4m3* p) { return reinterpret_cast<uint8_t*>(p); }

void fp8_quantize_per_tensor(const float* src, fp8_e4m3* dst, float* scale_out, int64_t n) {
    bool any_host = false;
    ARG(float, s, src, sz(n), In); ARG(uint8_t, d, bytes(dst), sz(n), Out); ARG(float, sc, scale_out, 1, Out);
    check(lhb_fp8_quantize_per_tensor(context(), s.get(), d.get(), sc.get(), n, g_stream), "fp8_quantize_per_tensor");
    d.writeback(); sc.writeback(); finish(any_host);
}

void fp8_quantize_per_row(const float* src, fp8_e4m3* dst, float* scales_out, int rows, int dim) {
    bool any_host = false;
    ARG(float, s, src, sz(rows, dim), In); ARG(uint8_t, d, bytes(dst), sz(rows, dim), Out); ARG(float, sc, scales_out, sz(rows), Out);
    check(lhb_fp8_quantize_per_row(context(), s.get(), d.get(), sc.get(), rows, dim, g_stream), "fp8_quantize_per_row");
    d.writeback(); sc.writeback(); finish(any_host);
}

void fp8_quantize_per_col(const float* src, fp8_e4m3* dst, float* scales_out, int rows, int cols) {
    bool any_host = false;
    ARG(float, s, src, sz(rows, cols), In); ARG(uint8_t, d, bytes(dst), sz(rows, cols), Out); ARG(float, sc, scales_out, sz(cols), Out);
    check(lhb_fp8_quantize_per_col(context(), s.get(), d.get(), sc.get(), rows, cols, g_stream), "fp8_quantize_per_col");
    d.writeback(); sc.writeback(); finish(any_host);
}

// dst = float(q) * scale with one scale (given by value), one per row or one per column
static void fp8_dequantize_any(const fp8_e4m3* src, const float* scales, size_t n_scales, bool scales_by_value,
                               float* dst, int rows, int cols, int mode, const char* where) {
    bool any_host = false;
    ARG(uint8_t, s, bytes(src), sz(rows, cols), In); ARG(float, d, dst, sz(rows, cols), Out);
    if (scales_by_value) {
        float* dsc = nullptr;                             // the C ABI reads the scale from device memory
        cuda_ok(cudaMalloc(&dsc, sizeof(float)), "cudaMalloc(scale)");
        cuda_ok(cudaMemcpyAsync(dsc, scales, sizeof(float), cudaMemcpyHostToDevice, g_stream), "H2D(scale)");
        const int e = lhb_fp8_dequantize(context(), s.get(), dsc, d.get(), rows, cols, mode, g_stream);
        cuda_ok(cudaStreamSynchronize(g_stream), "synchronize");
        cudaFree(dsc);
        check(e, where);
    } else {
        ARG(float, sc, scales, n_scales, In);
        check(lhb_fp8_dequantize(context(), s.get(), sc.get(), d.get(), rows, cols, mode, g_stream), where);
    }
    d.writeback(); finish(any_host);
}

void fp8_dequantize_per_tensor(const fp8_e4m3* src, float scale, float* dst, int64_t n) {
    // the C ABI takes rows x cols as ints: a long buffer is cut into rows of 2^20
    int64_t done = 0;
    while (done < n) {
        const int64_t part = std::min<int64_t>(n - done, int64_t(1) << 30);
        const int cols = static_cast<int>(std::min<int64_t>(part, 1 << 20));
        const int rows = static_cast<int>(part / cols);
        fp8_dequantize_any(src + done, &scale, 1, true, dst + done, rows, cols, 0, "fp8_dequantize_per_tensor");
        done += static_cast<int64_t>(rows) * cols;
    }
}

void fp8_dequantize_per_row(const fp8_e4m3* src, const float* scales, float* dst, int rows, int dim) {
    fp8_dequantize_any(src, scales, sz(rows), false, dst, rows, dim, 1, "fp8_dequantize_per_row");
}

void fp8_dequantize_per_col(const fp8_e4m3* src, const float* scales, float* dst, int rows, int cols) {
    fp8_dequantize_any(src, scales, sz(cols), false, dst, rows, cols, 2, "fp8_dequantize_per_col");
}

void gemm_fp8_e4m3(const fp8_e4m3* A, const fp8_e4m3* B, float A_scale, float B_scale, float* C, int M, int N, int K,
                   float alpha, float beta) {
    bool any_host = false;
    ARG(uint8_t, a, bytes(A), sz(M, K), In); ARG(uint8_t, b, bytes(B), sz(K, N), In);
    Arg<float> c(C, sz(M, N), beta == 0.0f ? Arg<float>::Out : Arg<float>::InOut, any_host);
    check(lhb_gemm_fp8_e4m3(context(), a.get(), b.get(), A_scale, B_scale, c.get(), M, N, K, alpha, beta, g_stream),
          "gemm_fp8_e4m3");
    c.writeback(); finish(any_host);
}

void q8_quantize_per_row(const float* src, int8_t* dst, float* scales_out, int rows, int dim) {
    bool any_host = false;
    ARG(float, s, src, sz(rows, dim), In); ARG(int8_t, d, dst, sz(rows, dim), Out); ARG(float, sc, scales_out, sz(rows), Out);
    check(lhb_q8_quantize_per_row(context(), s.get(), d.get(), sc.get(), rows, dim, g_stream), "q8_quantize_per_row");
    d.writeback(); sc.writeback(); finish(any_host);
}

void q8_dequantize_per_row(const int8_t* src, const float* scales, float* dst, int rows, int dim) {
    bool any_host = false;
    ARG(int8_t, s, src, sz(rows, dim), In); ARG(float, sc, scales, sz(rows), In); ARG(float, d, dst, sz(rows, dim), Out);
    check(lhb_q8_dequantize_per_row(context(), s.get(), sc.get(), d.get(), rows, dim, g_stream), "q8_dequantize_per_row");
    d.writeback(); finish(any_host);
}

void q8_quantize_per_col(const float* src, int8_t* dst, float* scales_out, int rows, int cols) {
    bool any_host = false;
    ARG(float, s, src, sz(rows, cols), In); ARG(int8_t, d, dst, sz(rows, cols), Out); ARG(float, sc, scales_out, sz(cols), Out);
    check(lhb_q8_quantize_per_col(context(), s.get(), d.get(), sc.get(), rows, cols, g_stream), "q8_quantize_per_col");
    d.writeback(); sc.writeback(); finish(any_host);
}

void q8_dequantize_per_col(const int8_t* src, const float* scales, float* dst, int rows, int cols) {
    bool any_host = false;
    ARG(int8_t, s, src, sz(rows, cols), In); ARG(float, sc, scales, sz(cols), In); ARG(float, d, dst, sz(rows, cols), Out);
    check(lhb_q8_dequantize_per_col(context(), s.get(), sc.get(), d.get(), rows, cols, g_stream), "q8_dequantize_per_col");
    d.writeback(); finish(any_host);
}

void q4_quantize_groupwise(const float* src, uint8_t* packed, float* scales_out, int K, int N, int G) {
    bool any_host = false;
    ARG(float, s, src, sz(K, N), In); ARG(uint8_t, p, packed, sz(K / 2, N), Out);
    ARG(float, sc, scales_out, sz(G > 0 ? K / G : 0, N), Out);
    check(lhb_q4_quantize_groupwise(context(), s.get(), p.get(), sc.get(), K, N, G, g_stream), "q4_quantize_groupwise");
    p.writeback(); sc.writeback(); finish(any_host);
}

void q4_dequantize_groupwise(const uint8_t* packed, const float* scales, float* dst, int K, int N, int G) {
    bool any_host = false;
    ARG(uint8_t, p, packed, sz(K / 2, N), In); ARG(float, sc, scales, sz(G > 0 ? K / G : 0, N), In);
    ARG(float, d, dst, sz(K, N), Out);
    check(lhb_q4_dequantize_groupwise(context(), p.get(), sc.get(), d.get(), K, N, G, g_stream), "q4_dequantize_groupwise");
    d.writeback(); finish(any_host);
}

void gemm_w8a8(const int8_t* A_q, const int8_t* B_q, const float* A_scales, const float* B_scales, float* C,
               int M, int N, int K, float alpha, float beta) {
    bool any_host = false;
    ARG(int8_t, a, A_q, sz(M, K), In); ARG(int8_t, b, B_q, sz(K, N), In);
    ARG(float, as, A_scales, sz(M), In); ARG(float, bs, B_scales, sz(N), In);
    Arg<float> c(C, sz(M, N), beta == 0.0f ? Arg<float>::Out : Arg<float>::InOut, any_host);
    check(lhb_gemm_w8a8(context(), a.get(), b.get(), as.get(), bs.get(), c.get(), M, N, K, alpha, beta, g_stream),
          "gemm_w8a8");
    c.writeback(); finish(any_host);
}

void gemm_w4a16_groupwise(const float* A, const uint8_t* B_packed, const float* B_scales, float* C, int M,
                          int N, int K, int G, float alpha, float beta) {
    bool any_host = false;
    ARG(float, a, A, sz(M, K), In); ARG(uint8_t, b, B_packed, sz(K / 2, N), In);
    ARG(float, bs, B_scales, sz(G > 0 ? K / G : 0, N), In);
    Arg<float> c(C, sz(M, N), beta == 0.0f ? Arg<float>::Out : Arg<float>::InOut, any_host);
    check(lhb_gemm_w4a16_groupwise(context(), a.get(), b.get(), bs.get(), c.get(), M, N, K, G, alpha, beta, g_stream),
          "gemm_w4a16_groupwise");
    c.writeback(); finish(any_host);
}

void gemm_w8a16_perchannel(const float* A, const int8_t* B_q, const float* B_scales, float* C, int M, int N,
                           int K, float alpha, float beta) {
    bool any_host = false;
    ARG(float, a, A, sz(M, K), In); ARG(int8_t, b, B_q, sz(K, N), In); ARG(float, bs, B_scales, sz(N), In);
    Arg<float> c(C, sz(M, N), beta == 0.0f ? Arg<float>::Out : Arg<float>::InOut, any_host);
    check(lhb_gemm_w8a16_perchannel(context(), a.get(), b.get(), bs.get(), c.get(), M, N, K, alpha, beta, g_stream),
          "gemm_w8a16_perchannel");
    c.writeback(); finish(any_host);
}

void paged_kv_append(float* k_pool, float* v_pool, const float* k_new, const float* v_new,
                     const int32_t* block_table, const PagedCacheLayout& L, int past_len, int seq_new) {
    if (seq_new <= 0) return;
    bool any_host = false;
    const lhb_paged_layout cl = to_c(L);
    const size_t nb = sz((past_len + seq_new + L.block_size - 1) / L.block_size);
    ARG(float, kp, k_pool, pool_elems(L), InOut); ARG(float, vp, v_pool, pool_elems(L), InOut);
    ARG(float, kn, k_new, sz(L.n_kv_heads, seq_new, L.head_dim), In);
    ARG(float, vn, v_new, sz(L.n_kv_heads, seq_new, L.head_dim), In);
    ARG(int32_t, bt, block_table, nb, In);
    check(lhb_paged_kv_append_f32(context(), kp.get(), vp.get(), kn.get(), vn.get(), bt.get(), &cl, past_len, seq_new,
                                  g_stream), "paged_kv_append");
    kp.writeback(); vp.writeback(); finish(any_host);
}

void paged_kv_append_q8(int8_t* k_pool, int8_t* v_pool, float* k_scales, float* v_scales, const float* k_new,
                        const float* v_new, const int32_t* block_table, const PagedCacheLayout& L,
                        int past_len, int seq_new) {
    if (seq_new <= 0) return;
    bool any_host = false;
    const lhb_paged_layout cl = to_c(L);
    const size_t nb = sz((past_len + seq_new + L.block_size - 1) / L.block_size);
    ARG(int8_t, kp, k_pool, pool_elems(L), InOut); ARG(int8_t, vp, v_pool, pool_elems(L), InOut);
    ARG(float, ks, k_scales, scale_elems(L), InOut); ARG(float, vs, v_scales, scale_elems(L), InOut);
    ARG(float, kn, k_new, sz(L.n_kv_heads, seq_new, L.head_dim), In);
    ARG(float, vn, v_new, sz(L.n_kv_heads, seq_new, L.head_dim), In);
    ARG(int32_t, bt, block_table, nb, In);
    check(lhb_paged_kv_append_q8(context(), kp.get(), vp.get(), ks.get(), vs.get(), kn.get(), vn.get(), bt.get(), &cl,
                                 past_len, seq_new, g_stream), "paged_kv_append_q8");
    kp.writeback(); vp.writeback(); ks.writeback(); vs.writeback(); finish(any_host);
}

void paged_attention_q8_batched(const float* Q, const int8_t* K_pool, const int8_t* V_pool, const float* K_scales,
                                const float* V_scales, const int32_t* block_tables, int max_blocks_per_req,
                                const int32_t* seq_lens, int n_requests, float* O, const PagedAttnConfig& cfg,
                                const PagedCacheLayout& L) {
    bool any_host = false;
    const lhb_paged_layout cl = to_c(L);
    const lhb_paged_attn_cfg cc = to_c(cfg);
    const size_t qn = sz(static_cast<int64_t>(n_requests) * cfg.n_q_heads, cfg.seq_q, cfg.head_dim);
    ARG(float, q, Q, qn, In); ARG(int8_t, kp, K_pool, pool_elems(L), In); ARG(int8_t, vp, V_pool, pool_elems(L), In);
    ARG(float, ks, K_scales, scale_elems(L), In); ARG(float, vs, V_scales, scale_elems(L), In);
    ARG(int32_t, bt, block_tables, sz(n_requests, max_blocks_per_req), In); ARG(int32_t, sl, seq_lens, sz(n_requests), In);
    ARG(float, o, O, qn, Out);
    check(lhb_paged_attention_q8_batched(context(), q.get(), kp.get(), vp.get(), ks.get(), vs.get(), bt.get(),
                                         max_blocks_per_req, sl.get(), n_requests, o.get(), &cc, &cl, g_stream),
          "paged_attention_q8_batched");
    o.writeback(); finish(any_host);
}

void paged_attention_q8(const float* Q, const int8_t* K_pool, const int8_t* V_pool, const float* K_scales,
                        const float* V_scales, const int32_t* block_table, int seq_len, float* O,
                        const PagedAttnConfig& cfg, const PagedCacheLayout& L) {
    bool any_host = false;
    const lhb_paged_layout cl = to_c(L);
    const lhb_paged_attn_cfg cc = to_c(cfg);
    const size_t qn = sz(cfg.n_q_heads, cfg.seq_q, cfg.head_dim);
    const size_t nb = sz((seq_len + L.block_size - 1) / L.block_size);
    ARG(float, q, Q, qn, In); ARG(int8_t, kp, K_pool, pool_elems(L), In); ARG(int8_t, vp, V_pool, pool_elems(L), In);
    ARG(float, ks, K_scales, scale_elems(L), In); ARG(float, vs, V_scales, scale_elems(L), In);
    ARG(int32_t, bt, block_table, nb, In); ARG(float, o, O, qn, Out);
    check(lhb_paged_attention_q8(context(), q.get(), kp.get(), vp.get(), ks.get(), vs.get(), bt.get(), seq_len, o.get(),
                                 &cc, &cl, g_stream), "paged_attention_q8");
    o.writeback(); finish(any_host);
}

void paged_attention_batched(const float* Q, const float* K_pool, const float* V_pool, const int32_t* block_tables,
                             int max_blocks_per_req, const int32_t* seq_lens, int n_requests, float* O,
                             const PagedAttnConfig& cfg, const PagedCacheLayout& L) {
    bool any_host = false;
    const lhb_paged_layout cl = to_c(L);
    const lhb_paged_attn_cfg cc = to_c(cfg);
    const size_t qn = sz(static_cast<int64_t>(n_requests) * cfg.n_q_heads, cfg.seq_q, cfg.head_dim);
    ARG(float, q, Q, qn, In); ARG(float, kp, K_pool, pool_elems(L), In); ARG(float, vp, V_pool, pool_elems(L), In);
    ARG(int32_t, bt, block_tables, sz(n_requests, max_blocks_per_req), In); ARG(int32_t, sl, seq_lens, sz(n_requests), In);
    ARG(float, o, O, qn, Out);
    check(lhb_paged_attention_f32_batched(context(), q.get(), kp.get(), vp.get(), bt.get(), max_blocks_per_req, sl.get(),
                                          n_requests, o.get(), &cc, &cl, g_stream), "paged_attention_batched");
    o.writeback(); finish(any_host);
}

void paged_attention(const float* Q, const float* K_pool, const float* V_pool, const int32_t* block_table,
                     int seq_len, float* O, const PagedAttnConfig& cfg, const PagedCacheLayout& L) {
    // one request = a batch of one whose table has ceil(seq_len / block_size) entries
    bool any_host = false;
    const int nb = seq_len > 0 ? (seq_len + L.block_size - 1) / L.block_size : 1;
    ARG(int32_t, sl, &seq_len, 1, In);
    (void)any_host;
    paged_attention_batched(Q, K_pool, V_pool, block_table, nb, sl.get(), 1, O, cfg, L);
}

namespace b200 {

void rmsnorm(const float* x, const float* gamma, float* y, int rows, int dim, float eps) {
    bool any_host = false;
    ARG(float, xi, x, sz(rows, dim), In); ARG(float, g, gamma, sz(dim), In); ARG(float, yo, y, sz(rows, dim), Out);
    check(lhb_rmsnorm(context(), xi.get(), g.get(), yo.get(), rows, dim, eps, g_stream), "rmsnorm");
    yo.writeback(); finish(any_host);
}

void rope(float* x, int seq, int n_heads, int head_dim, float theta_base, float freq_scale, bool interleaved,
          int pos_offset) {
    bool any_host = false;
    ARG(float, xi, x, sz(seq, n_heads) * head_dim, InOut);
    check(lhb_rope(context(), xi.get(), seq, n_heads, head_dim, theta_base, freq_scale, interleaved ? 1 : 0, pos_offset,
                   g_stream), "rope");
    xi.writeback(); finish(any_host);
}

void swiglu(const float* x, float* y, int rows, int dim) {
    bool any_host = false;
    ARG(float, xi, x, sz(rows, dim) * 2, In); ARG(float, yo, y, sz(rows, dim), Out);
    check(lhb_swiglu(context(), xi.get(), yo.get(), rows, dim, g_stream), "swiglu");
    yo.writeback(); finish(any_host);
}

}  // namespace b200

}  // namespace lh

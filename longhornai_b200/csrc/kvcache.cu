// Paged KV-cache append kernels.
//
// Pools follow the reference layout [num_blocks, n_kv_heads, block_size,
// head_dim] with one fp32 scale per (block, head, slot) row
// (src/kernels/kvcache.hpp:34-41, src/kernels/kvcache_quant.hpp:31-36).  New
// rows arrive head-major [n_kv_heads, seq_new, head_dim].  One warp quantises
// one (token, head) row of K and of V: shuffle max|x|, scale = max/127 (1 for a
// zero row), q = sat(x * (1/scale)) -- the reciprocal-multiply idiom of
// src/kernels/kvcache_quant.cpp:24-35, reproduced bit-for-bit.
#include "common.cuh"

namespace lhb {

__device__ __forceinline__ void quantize_row_warp(const float* __restrict__ x,
                                                  int8_t* __restrict__ q,
                                                  float* __restrict__ scale_out, int d, int lane) {
    float m = 0.0f;
    for (int i = lane; i < d; i += 32) m = fmaxf(m, fabsf(x[i]));
    m = warp_max(m);
    const float scale = (m > 0.0f) ? __fdiv_rn(m, 127.0f) : 1.0f;
    const float inv = __fdiv_rn(1.0f, scale);
    if ((d & 3) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(q)) & 15) == 0) {
        // 4 values per lane per step: one 128-bit load, one 32-bit store
        for (int i = lane * 4; i < d; i += 128) {
            const float4 v = *reinterpret_cast<const float4*>(x + i);
            char4 o;
            o.x = static_cast<signed char>(sat_rne(__fmul_rn(v.x, inv), 127));
            o.y = static_cast<signed char>(sat_rne(__fmul_rn(v.y, inv), 127));
            o.z = static_cast<signed char>(sat_rne(__fmul_rn(v.z, inv), 127));
            o.w = static_cast<signed char>(sat_rne(__fmul_rn(v.w, inv), 127));
            *reinterpret_cast<char4*>(q + i) = o;
        }
    } else {
        for (int i = lane; i < d; i += 32) q[i] = static_cast<int8_t>(sat_rne(__fmul_rn(x[i], inv), 127));
    }
    if (lane == 0) *scale_out = scale;
}

// grid.x covers (request, token, head) rows, 4 warps per CTA.  past_lens ==
// nullptr means a single request with the scalar past_len.
__global__ void __launch_bounds__(128)
paged_kv_append_q8_kernel(int8_t* __restrict__ k_pool, int8_t* __restrict__ v_pool,
                          float* __restrict__ k_scales, float* __restrict__ v_scales,
                          const float* __restrict__ k_new, const float* __restrict__ v_new,
                          const int32_t* __restrict__ block_tables, int max_blocks,
                          const int32_t* __restrict__ past_lens, int past_len_scalar, int n_req,
                          int seq_new, lhb_paged_layout L) {
    const int lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * 4 + (threadIdx.x >> 5);
    const int64_t total = static_cast<int64_t>(n_req) * seq_new * L.n_kv_heads;
    if (row >= total) return;
    const int h = static_cast<int>(row % L.n_kv_heads);
    const int s = static_cast<int>((row / L.n_kv_heads) % seq_new);
    const int r = static_cast<int>(row / (static_cast<int64_t>(L.n_kv_heads) * seq_new));
    const int past = past_lens ? past_lens[r] : past_len_scalar;
    const int pos = past + s;
    // A position the request's table row cannot describe (negative, or at or past max_blocks *
    // block_size where the row width is known) writes nothing: the next table entry would be
    // another request's page.
    if (pos < 0 || (past_lens && pos / L.block_size >= max_blocks)) return;
    const int blk = block_tables[static_cast<int64_t>(r) * max_blocks + pos / L.block_size];
    if (blk < 0 || blk >= L.num_blocks) return;   // unallocated page: nothing to write
    const int slot = pos % L.block_size;
    const int64_t srow = (static_cast<int64_t>(blk) * L.n_kv_heads + h) * L.block_size + slot;
    const int64_t src = ((static_cast<int64_t>(r) * L.n_kv_heads + h) * seq_new + s) * L.head_dim;
    quantize_row_warp(k_new + src, k_pool + srow * L.head_dim, k_scales + srow, L.head_dim, lane);
    quantize_row_warp(v_new + src, v_pool + srow * L.head_dim, v_scales + srow, L.head_dim, lane);
}

// Decode-step fusion: the fused QKV projection's output row [q heads | k heads | v heads]
// is split, the q and k heads are rotated (rotary embedding at the request's position), q goes
// to a contiguous [n_req, n_q_heads, head_dim] tensor and the rotated k and the v rows are
// quantised straight into the request's page.  One warp per (request, head); the result is
// bit-identical to rope on q, rope on k and paged_kv_append_q8 run one after the other
// (src/kernels/rope.cpp:47-86, src/kernels/kvcache_quant.cpp:58-80), without the three
// intermediate tensors and five launches.
constexpr int QKV_MAX_D = 256;

__global__ void __launch_bounds__(128)
qkv_rope_append_q8_kernel(const float* __restrict__ qkv, int64_t row_stride, float* __restrict__ q_out,
                          int8_t* __restrict__ k_pool, int8_t* __restrict__ v_pool, float* __restrict__ k_scales,
                          float* __restrict__ v_scales, const int32_t* __restrict__ block_tables, int max_blocks,
                          const int32_t* __restrict__ positions, int n_req, int n_q_heads, lhb_paged_layout L,
                          float theta_base, float freq_scale, int interleaved) {
    __shared__ __align__(16) float rot[4][QKV_MAX_D];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int heads = n_q_heads + 2 * L.n_kv_heads;
    const int64_t item = static_cast<int64_t>(blockIdx.x) * 4 + w;
    if (item >= static_cast<int64_t>(n_req) * heads) return;
    const int r = static_cast<int>(item / heads), j = static_cast<int>(item % heads);
    const int d = L.head_dim, half = d >> 1;
    const int pos = positions[r];
    const float* src = qkv + r * row_stride + static_cast<int64_t>(j) * d;
    const bool is_v = j >= n_q_heads + L.n_kv_heads;
    const float* row = src;
    if (!is_v) {
        for (int i = lane; i < half; i += 32) {
            float sn, c;
            rope_sincos(pos, i, d, theta_base, freq_scale, &sn, &c);
            const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + half;
            const float a = src[ia], b = src[ib];
            rot[w][ia] = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, sn));
            rot[w][ib] = interleaved ? __fadd_rn(__fmul_rn(a, sn), __fmul_rn(b, c))
                                     : __fadd_rn(__fmul_rn(b, c), __fmul_rn(a, sn));
        }
        __syncwarp();
        row = rot[w];
    }
    if (j < n_q_heads) {
        float* dst = q_out + (static_cast<int64_t>(r) * n_q_heads + j) * d;
        for (int i = lane; i < d; i += 32) dst[i] = row[i];
        return;
    }
    const int h = is_v ? j - n_q_heads - L.n_kv_heads : j - n_q_heads;
    if (pos < 0 || pos / L.block_size >= max_blocks) return;      // outside the request's table row: nothing to write
    const int blk = block_tables[static_cast<int64_t>(r) * max_blocks + pos / L.block_size];
    if (blk < 0 || blk >= L.num_blocks) return;       // unallocated page: nothing to write
    const int64_t srow = (static_cast<int64_t>(blk) * L.n_kv_heads + h) * L.block_size + pos % L.block_size;
    if (is_v) quantize_row_warp(row, v_pool + srow * d, v_scales + srow, d, lane);
    else quantize_row_warp(row, k_pool + srow * d, k_scales + srow, d, lane);
}

// fp32 append (src/kernels/kvcache.cpp:7-32): a row copy.
__global__ void __launch_bounds__(128)
paged_kv_append_f32_kernel(float* __restrict__ k_pool, float* __restrict__ v_pool,
                           const float* __restrict__ k_new, const float* __restrict__ v_new,
                           const int32_t* __restrict__ block_table, int past_len, int seq_new,
                           lhb_paged_layout L) {
    const int lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * 4 + (threadIdx.x >> 5);
    if (row >= static_cast<int64_t>(seq_new) * L.n_kv_heads) return;
    const int h = static_cast<int>(row % L.n_kv_heads);
    const int s = static_cast<int>(row / L.n_kv_heads);
    const int pos = past_len + s;
    const int blk = block_table[pos / L.block_size];
    if (blk < 0 || blk >= L.num_blocks) return;
    const int64_t dst = ((static_cast<int64_t>(blk) * L.n_kv_heads + h) * L.block_size +
                         pos % L.block_size) * L.head_dim;
    const int64_t src = (static_cast<int64_t>(h) * seq_new + s) * L.head_dim;
    for (int i = lane; i < L.head_dim; i += 32) {
        k_pool[dst + i] = k_new[src + i];
        v_pool[dst + i] = v_new[src + i];
    }
}

}  // namespace lhb

using namespace lhb;

static int check_layout(const lhb_paged_layout* L) {
    if (!L) return LHB_ERR_NULL;
    if (L->num_blocks <= 0 || L->block_size <= 0 || L->n_kv_heads <= 0 || L->head_dim <= 0)
        return LHB_ERR_BAD_SHAPE;
    return LHB_OK;
}

extern "C" {

int lhb_paged_kv_append_q8(lhb_ctx* ctx, int8_t* k_pool, int8_t* v_pool, float* k_scales,
                           float* v_scales, const float* k_new, const float* v_new,
                           const int32_t* block_table, const lhb_paged_layout* layout, int past_len,
                           int seq_new, void* stream) {
    if (!ctx || !k_pool || !v_pool || !k_scales || !v_scales || !block_table) return LHB_ERR_NULL;
    if (int e = check_layout(layout)) return e;
    if (seq_new <= 0) return LHB_OK;                 // reference: early return
    if (!k_new || !v_new) return LHB_ERR_NULL;
    if (past_len < 0) return LHB_ERR_BAD_SHAPE;
    const int64_t rows = static_cast<int64_t>(seq_new) * layout->n_kv_heads;
    paged_kv_append_q8_kernel<<<static_cast<unsigned>(ceil_div64(rows, 4)), 128, 0,
                                as_stream(stream)>>>(k_pool, v_pool, k_scales, v_scales, k_new,
                                                     v_new, block_table, 0, nullptr, past_len, 1,
                                                     seq_new, *layout);
    LHB_LAUNCH_CHECK();
    return LHB_OK;
}

int lhb_paged_kv_append_q8_batched(lhb_ctx* ctx, int8_t* k_pool, int8_t* v_pool, float* k_scales,
                                   float* v_scales, const float* k_new, const float* v_new,
                                   const int32_t* block_tables, int max_blocks_per_req,
                                   const int32_t* past_lens, int n_requests,
                                   const lhb_paged_layout* layout, int seq_new, void* stream) {
    if (!ctx || !k_pool || !v_pool || !k_scales || !v_scales || !block_tables || !past_lens)
        return LHB_ERR_NULL;
    if (int e = check_layout(layout)) return e;
    if (n_requests < 0 || max_blocks_per_req <= 0) return LHB_ERR_BAD_SHAPE;
    if (seq_new <= 0 || n_requests == 0) return LHB_OK;
    if (!k_new || !v_new) return LHB_ERR_NULL;
    const int64_t rows = static_cast<int64_t>(n_requests) * seq_new * layout->n_kv_heads;
    paged_kv_append_q8_kernel<<<static_cast<unsigned>(ceil_div64(rows, 4)), 128, 0,
                                as_stream(stream)>>>(k_pool, v_pool, k_scales, v_scales, k_new,
                                                     v_new, block_tables, max_blocks_per_req,
                                                     past_lens, 0, n_requests, seq_new, *layout);
    LHB_LAUNCH_CHECK();
    return LHB_OK;
}

int lhb_paged_kv_append_f32(lhb_ctx* ctx, float* k_pool, float* v_pool, const float* k_new,
                            const float* v_new, const int32_t* block_table,
                            const lhb_paged_layout* layout, int past_len, int seq_new,
                            void* stream) {
    if (!ctx || !k_pool || !v_pool || !block_table) return LHB_ERR_NULL;
    if (int e = check_layout(layout)) return e;
    if (seq_new <= 0) return LHB_OK;
    if (!k_new || !v_new) return LHB_ERR_NULL;
    if (past_len < 0) return LHB_ERR_BAD_SHAPE;
    const int64_t rows = static_cast<int64_t>(seq_new) * layout->n_kv_heads;
    paged_kv_append_f32_kernel<<<static_cast<unsigned>(ceil_div64(rows, 4)), 128, 0,
                                 as_stream(stream)>>>(k_pool, v_pool, k_new, v_new, block_table,
                                                      past_len, seq_new, *layout);
    LHB_LAUNCH_CHECK();
    return LHB_OK;
}

int lhb_qkv_rope_append_q8_decode(lhb_ctx* ctx, const float* qkv, int64_t row_stride, float* q_out, int8_t* k_pool,
                                  int8_t* v_pool, float* k_scales, float* v_scales, const int32_t* block_tables,
                                  int max_blocks_per_req, const int32_t* positions, int n_requests, int n_q_heads,
                                  const lhb_paged_layout* layout, float theta_base, float freq_scale,
                                  int interleaved, void* stream) {
    if (!ctx || !qkv || !q_out || !k_pool || !v_pool || !k_scales || !v_scales || !block_tables || !positions)
        return LHB_ERR_NULL;
    if (int e = check_layout(layout)) return e;
    if (n_requests < 0 || n_q_heads <= 0 || max_blocks_per_req <= 0 || (layout->head_dim & 1)) return LHB_ERR_BAD_SHAPE;
    if (layout->head_dim > QKV_MAX_D) return LHB_ERR_UNSUPPORTED;
    const int heads = n_q_heads + 2 * layout->n_kv_heads;
    if (row_stride < static_cast<int64_t>(heads) * layout->head_dim) return LHB_ERR_BAD_SHAPE;
    if (n_requests == 0) return LHB_OK;
    const int64_t items = static_cast<int64_t>(n_requests) * heads;
    qkv_rope_append_q8_kernel<<<static_cast<unsigned>(ceil_div64(items, 4)), 128, 0, as_stream(stream)>>>(
        qkv, row_stride, q_out, k_pool, v_pool, k_scales, v_scales, block_tables, max_blocks_per_req, positions,
        n_requests, n_q_heads, *layout, theta_base, freq_scale, interleaved);
    LHB_LAUNCH_CHECK();
    return LHB_OK;
}

}  // extern "C"

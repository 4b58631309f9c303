// Generic paged attention: any head_dim, block_size, seq_q, causal / window /
// chunk masks, int8 pools with per-row scales or fp32 pools.
//
// One CTA per (request, query head, query row).  It keeps the reference's
// three-pass shape (src/kernels/kvcache_quant.cpp:82-161,
// src/kernels/paged_attention.cpp:36-108): scores + max, exp + sum, then the
// weighted V sum with p = e * (1/sum); only the order of the fp32 additions
// differs (lanes split head_dim, warps split keys).  The score row lives in
// shared memory, so the visible key range must fit in it; the decode fast
// path (paged_attention_decode.cu) has no such limit.
#include "common.cuh"

namespace lhb {

constexpr int PAG_THREADS = 128;

__device__ __forceinline__ bool key_visible(const lhb_paged_attn_cfg& c, int i, int j, int shift) {
    if (c.causal && j > shift + i) return false;
    if (c.window > 0 && j < shift + i - c.window + 1) return false;
    if (c.chunk > 0 && (shift + i) / c.chunk != j / c.chunk) return false;
    return true;
}

__device__ __forceinline__ float block_reduce(float v, float* red, bool is_max) {
    v = is_max ? warp_max(v) : warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = red[0];
    for (int w = 1; w < PAG_THREADS / 32; ++w) r = is_max ? fmaxf(r, red[w]) : r + red[w];
    return r;
}

template <bool Q8>
__global__ void __launch_bounds__(PAG_THREADS)
paged_attention_generic_kernel(const float* __restrict__ Q, const void* __restrict__ Kp,
                               const void* __restrict__ Vp, const float* __restrict__ Ks,
                               const float* __restrict__ Vs, const int32_t* __restrict__ tables,
                               int max_blocks, const int32_t* __restrict__ seq_lens,
                               int seq_len_scalar, float* __restrict__ O, lhb_paged_attn_cfg cfg,
                               lhb_paged_layout L, float sm_scale, int smem_keys,
                               int* __restrict__ status) {
    extern __shared__ float scores[];
    __shared__ float red[PAG_THREADS / 32];
    const int i = blockIdx.x, h = blockIdx.y, r = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int d = cfg.head_dim, B = L.block_size;
    const int kvh = h / (cfg.n_q_heads / cfg.n_kv_heads);
    int seq_len = seq_lens ? seq_lens[r] : seq_len_scalar;
    seq_len = max(0, min(seq_len, max_blocks * B));
    const int shift = seq_len - cfg.seq_q;
    const int32_t* table = tables + static_cast<int64_t>(r) * max_blocks;
    const int64_t qo = ((static_cast<int64_t>(r) * cfg.n_q_heads + h) * cfg.seq_q + i) * d;
    const float* q = Q + qo;
    float* o = O + qo;

    int last = seq_len - 1;
    if (cfg.causal) last = min(last, shift + i);
    int first = 0;
    if (cfg.window > 0) first = max(0, shift + i - cfg.window + 1);
    if (cfg.chunk > 0) first = max(first, ((shift + i) / cfg.chunk) * cfg.chunk);
    const int n_keys = last - first + 1;
    if (n_keys <= 0 || n_keys > smem_keys) {
        // no visible key: zeros, as in the reference.  A key range longer than
        // the shared score row is reported through the status word.
        if (n_keys > smem_keys && threadIdx.x == 0) atomicExch(status, LHB_ERR_UNSUPPORTED);
        for (int t = threadIdx.x; t < d; t += PAG_THREADS) o[t] = 0.0f;
        return;
    }

    // pass 1: scores and running max
    float mx = -INFINITY;
    for (int j = first + warp; j <= last; j += PAG_THREADS / 32) {
        float s = -INFINITY;
        // A table entry outside the pool (the cache manager's -1 for a page that was never
        // allocated or has been released) masks its keys, as in the decode kernel: the key gets
        // no weight and its page is never dereferenced, in this pass or in the third.
        const int blk = table[j / B];
        if (blk >= 0 && blk < L.num_blocks && key_visible(cfg, i, j, shift)) {
            const int64_t row = (static_cast<int64_t>(blk) * L.n_kv_heads + kvh) * B + j % B;
            float dot = 0.0f;
            if (Q8) {
                const int8_t* k = static_cast<const int8_t*>(Kp) + row * d;
                const float ks = Ks[row];
                for (int t = lane; t < d; t += 32) dot = fmaf(q[t], static_cast<float>(k[t]) * ks, dot);
            } else {
                const float* k = static_cast<const float*>(Kp) + row * d;
                for (int t = lane; t < d; t += 32) dot = fmaf(q[t], k[t], dot);
            }
            s = warp_sum(dot) * sm_scale;
        }
        if (lane == 0) scores[j - first] = s;
        mx = fmaxf(mx, s);
    }
    mx = block_reduce(mx, red, true);
    if (mx == -INFINITY) {
        for (int t = threadIdx.x; t < d; t += PAG_THREADS) o[t] = 0.0f;
        return;
    }
    // pass 2: exponentials and their sum
    float sum = 0.0f;
    for (int j = threadIdx.x; j < n_keys; j += PAG_THREADS) {
        const float e = expf(scores[j] - mx);   // masked keys hold -inf -> 0
        scores[j] = e;
        sum += e;
    }
    sum = block_reduce(sum, red, false);
    const float inv = 1.0f / sum;
    // pass 3: weighted sum of V rows; a thread owns output elements t
    for (int t = threadIdx.x; t < d; t += PAG_THREADS) {
        float acc = 0.0f;
        for (int j = 0; j < n_keys; ++j) {
            const float p = scores[j] * inv;
            if (p == 0.0f) continue;
            const int pos = first + j;
            const int blk = table[pos / B];
            const int64_t row = (static_cast<int64_t>(blk) * L.n_kv_heads + kvh) * B + pos % B;
            if (Q8)
                acc = fmaf(p, static_cast<float>(static_cast<const int8_t*>(Vp)[row * d + t]) * Vs[row], acc);
            else
                acc = fmaf(p, static_cast<const float*>(Vp)[row * d + t], acc);
        }
        o[t] = acc;
    }
}

int launch_paged_attention_generic(lhb_ctx* ctx, bool q8, const float* Q, const void* Kp,
                                   const void* Vp, const float* Ks, const float* Vs,
                                   const int32_t* tables, int max_blocks, const int32_t* seq_lens,
                                   int seq_len_scalar, int n_req, float* O,
                                   const lhb_paged_attn_cfg& cfg, const lhb_paged_layout& L,
                                   cudaStream_t st) {
    const float sm_scale = cfg.scale > 0.0f ? cfg.scale : 1.0f / sqrtf(static_cast<float>(cfg.head_dim));
    int64_t keys = static_cast<int64_t>(max_blocks) * L.block_size;
    if (!seq_lens) keys = seq_len_scalar > 0 ? seq_len_scalar : 1;
    if (cfg.window > 0 && cfg.window < keys) keys = cfg.window;
    if (keys < 1) keys = 1;
    const size_t smem = static_cast<size_t>(keys) * sizeof(float);
    if (smem > 200 * 1024) return LHB_ERR_UNSUPPORTED;
    auto kern = q8 ? paged_attention_generic_kernel<true> : paged_attention_generic_kernel<false>;
    if (smem > 48 * 1024)
        LHB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(smem)));
    dim3 grid(cfg.seq_q, cfg.n_q_heads, n_req);
    kern<<<grid, PAG_THREADS, smem, st>>>(Q, Kp, Vp, Ks, Vs, tables, max_blocks, seq_lens,
                                          seq_len_scalar, O, cfg, L, sm_scale,
                                          static_cast<int>(keys), ctx->status_word);
    LHB_LAUNCH_CHECK();
    return LHB_OK;
}

}  // namespace lhb

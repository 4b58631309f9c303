/*
 * lhb200 -- C ABI of the B200 (sm_100a) implementation of LonghornAI's
 * quantized decode hot path.
 *
 * Every entry point mirrors one free function of the reference's
 * `namespace lh` kernel layer (the citation above each declaration gives the
 * reference header it replaces).  Differences that the GPU imposes, and that
 * are the same for every call:
 *
 *   - all data pointers are DEVICE pointers on the context's device;
 *   - the call only ENQUEUES work on `stream` (a cudaStream_t passed as
 *     void*; NULL = the legacy default stream) and never synchronises;
 *   - the first argument is a context created once per device, which owns the
 *     scratch arena the split kernels use, so no call allocates device memory;
 *   - the return value is 0 or a negative lhb_status; nothing throws.  The
 *     reference validates nothing and returns void; here shape and alignment
 *     preconditions are checked and reported.
 *
 * Alignment contract: base pointers 16-byte aligned.  Any shape is accepted;
 * shapes that meet the fast-path conditions documented per call run the
 * tensor-core kernels, others run a generic kernel with identical results
 * within the stated tolerance.
 *
 * There is no CPU fallback: without a CUDA device every compute call returns
 * LHB_ERR_CUDA.
 */
#ifndef LHB200_H
#define LHB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LHB_API __attribute__((visibility("default")))

typedef enum lhb_status {
    LHB_OK = 0,
    LHB_ERR_BAD_SHAPE = -1,    /* a dimension is non-positive or violates a precondition */
    LHB_ERR_MISALIGNED = -2,   /* a pointer misses the 16-byte alignment contract */
    LHB_ERR_UNSUPPORTED = -3,  /* valid in the reference, not implemented here */
    LHB_ERR_CUDA = -4,         /* a CUDA runtime/driver call failed (see lhb_last_error) */
    LHB_ERR_NULL = -5,         /* a required pointer (or the context) is NULL */
    LHB_ERR_SCRATCH = -6,      /* the context's scratch arena is too small for this call */
    LHB_ERR_TIMEOUT = -7       /* a bounded device-side wait gave up (read via lhb_ctx_poll) */
} lhb_status;

typedef struct lhb_ctx lhb_ctx;

/* Mirrors lh::PagedCacheLayout (src/kernels/kvcache.hpp:26-31): pools are
 * [num_blocks, n_kv_heads, block_size, head_dim], scale pools
 * [num_blocks, n_kv_heads, block_size]. */
typedef struct lhb_paged_layout {
    int num_blocks;
    int block_size;
    int n_kv_heads;
    int head_dim;
} lhb_paged_layout;

/* Mirrors lh::PagedAttnConfig (src/kernels/paged_attention.hpp:28-37);
 * `causal` is an int (0/1); scale <= 0 means 1/sqrt(head_dim). */
typedef struct lhb_paged_attn_cfg {
    int n_q_heads;
    int n_kv_heads;
    int seq_q;
    int head_dim;
    int causal;
    float scale;
    int window;
    int chunk;
} lhb_paged_attn_cfg;

/* ---- context ------------------------------------------------------------ */

/* Create the per-device context: a scratch arena of `scratch_bytes` (0 = the
 * 64 MiB default) and a device status word.  No counterpart in the reference
 * (its kernels use std::vector scratch: src/kernels/gemm_quant.cpp:59,
 * src/kernels/kvcache_quant.cpp:93). */
LHB_API int lhb_ctx_create(int device, size_t scratch_bytes, lhb_ctx** out);
LHB_API int lhb_ctx_destroy(lhb_ctx* ctx);
/* Persistent kernels of this context (the tensor-core GEMMs) use at most `sm_limit` SMs (0 = all):
 * a caller that runs its own communication kernels beside them keeps SMs free for those.  No
 * counterpart in the reference. */
LHB_API int lhb_ctx_set_sm_limit(lhb_ctx* ctx, int sm_limit);
/* Synchronise `stream` and return the device status word (0, or
 * LHB_ERR_TIMEOUT if a kernel's bounded wait expired); clears it.  After a
 * non-zero report the context's arrival counters are zeroed as well, so the
 * context stays usable (the results of the call that timed out are undefined). */
LHB_API int lhb_ctx_poll(lhb_ctx* ctx, void* stream);
LHB_API const char* lhb_status_string(int status);
/* Text of the last failing CUDA call on this thread ("" if none). */
LHB_API const char* lhb_last_error(void);
/* 1 when a W4/W8 GEMM or paged-attention call with these arguments takes the
 * tensor-core fast path, 0 when it takes the generic kernel (for tests and
 * benchmarks to state which path they timed). */
LHB_API int lhb_gemm_w4a16_fast_path(int M, int N, int K, int group_size);
LHB_API int lhb_gemm_w8a16_fast_path(int M, int N, int K);
LHB_API int lhb_gemm_w8a8_fast_path(int M, int N, int K);
LHB_API int lhb_paged_attention_q8_fast_path(const lhb_paged_attn_cfg* cfg,
                                             const lhb_paged_layout* layout);

/* ---- quantisers (bit-exact with the reference) ---------------------------- */

/* lh::q8_quantize_per_tensor / q8_dequantize_per_tensor (src/kernels/quant.hpp:31-34,
 * src/kernels/quant.cpp:33-54): one fp32 scale = max|x| / 127 (1 if 0) for the whole buffer,
 * q = sat(x * (1 / scale)).  `scale_out` is a device pointer; the dequantiser takes the scale by
 * value, as the reference does. */
LHB_API int lhb_q8_quantize_per_tensor(lhb_ctx* ctx, const float* src, int8_t* dst, float* scale_out,
                                       int64_t n, void* stream);
LHB_API int lhb_q8_dequantize_per_tensor(lhb_ctx* ctx, const int8_t* src, float scale, float* dst,
                                         int64_t n, void* stream);
/* lh::q8_quantize_per_row / q8_dequantize_per_row (src/kernels/quant.hpp:38-41). */
LHB_API int lhb_q8_quantize_per_row(lhb_ctx* ctx, const float* src, int8_t* dst,
                                    float* scales_out, int rows, int dim, void* stream);
LHB_API int lhb_q8_dequantize_per_row(lhb_ctx* ctx, const int8_t* src, const float* scales,
                                      float* dst, int rows, int dim, void* stream);
/* lh::q8_quantize_per_col / q8_dequantize_per_col (src/kernels/quant.hpp:45-48). */
LHB_API int lhb_q8_quantize_per_col(lhb_ctx* ctx, const float* src, int8_t* dst,
                                    float* scales_out, int rows, int cols, void* stream);
LHB_API int lhb_q8_dequantize_per_col(lhb_ctx* ctx, const int8_t* src, const float* scales,
                                      float* dst, int rows, int cols, void* stream);
/* lh::q4_quantize_groupwise / q4_dequantize_groupwise (src/kernels/quant.hpp:60-63).
 * K even, group_size divides K. */
LHB_API int lhb_q4_quantize_groupwise(lhb_ctx* ctx, const float* src, uint8_t* packed,
                                      float* scales_out, int K, int N, int group_size,
                                      void* stream);
LHB_API int lhb_q4_dequantize_groupwise(lhb_ctx* ctx, const uint8_t* packed, const float* scales,
                                        float* dst, int K, int N, int group_size, void* stream);

/* ---- quantized GEMMs ------------------------------------------------------- */

/* lh::gemm_w8a8 (src/kernels/gemm_quant.hpp:42-45): int8 A [M,K] x int8 B [K,N]
 * (N contiguous), int32 accumulate, C = beta*C + alpha*A_scales[m]*B_scales[n]*acc.
 * With beta == 0 the result is bit-identical to the reference. */
LHB_API int lhb_gemm_w8a8(lhb_ctx* ctx, const int8_t* A_q, const int8_t* B_q,
                          const float* A_scales, const float* B_scales, float* C, int M, int N,
                          int K, float alpha, float beta, void* stream);

/* N-sharded form of gemm_w8a8 across the GPUs of one machine (no counterpart in the reference,
 * which has no multi-device path; the arithmetic is src/kernels/gemm_quant.cpp:29-49 on a column
 * slab, which is self-contained: src/kernels/gemm_quant.hpp:35-45).  This rank holds B_q
 * [K, N_local] and B_scales [N_local]; full_C is a HOST array of `world` device pointers, entry r
 * the base of rank r's full-width fp32 matrix [M, N_local * world] as mapped in THIS process
 * (entry `rank` this rank's own, the others peer memory: cudaIpc / lhb_peer_open).  The kernel's
 * epilogue stores every finished tile into columns [rank * N_local, (rank + 1) * N_local) of all
 * `world` matrices (its own with plain stores, the peers' as TMA bulk stores of staged 32 x 32
 * pieces; LHB_W8A8_PUSH=st in the environment selects plain stores there too) while its main loop
 * continues, so the transfer over NVLink
 * overlaps the arithmetic tile by tile and every rank ends up with the row-major [M, N] result
 * without a gather or a re-layout.  beta is 0 (the slab is overwritten).  The stores of a rank are
 * complete when its stream has passed the call; a rank may read its matrix once every rank's
 * stream has (a stream-ordered collective, or a barrier after synchronising).  Only shapes of
 * lhb_gemm_w8a8_fast_path with N_local a multiple of 32; others return LHB_ERR_UNSUPPORTED (run
 * lhb_gemm_w8a8 and gather). */
LHB_API int lhb_gemm_w8a8_sharded(lhb_ctx* ctx, const int8_t* A_q, const int8_t* B_q, const float* A_scales,
                                  const float* B_scales, void* const* full_C, int rank, int world, int M,
                                  int N_local, int K, float alpha, void* stream);
/* lh::gemm_w4a16_groupwise (src/kernels/gemm_quant.hpp:54-57): fp32 A [M,K],
 * packed int4 B [K/2,N] with fp32 scales [K/G,N], fp32 C [M,N]. */
LHB_API int lhb_gemm_w4a16_groupwise(lhb_ctx* ctx, const float* A, const uint8_t* B_packed,
                                     const float* B_scales, float* C, int M, int N, int K,
                                     int group_size, float alpha, float beta, void* stream);
/* Weight-only int8 per-output-channel GEMM.  The reference has no single
 * function: it is q8_dequantize_per_col (src/kernels/quant.hpp:47) followed by
 * gemm (src/kernels/gemm.hpp:18); this call fuses the two. */
LHB_API int lhb_gemm_w8a16_perchannel(lhb_ctx* ctx, const float* A, const int8_t* B_q,
                                      const float* B_scales, float* C, int M, int N, int K,
                                      float alpha, float beta, void* stream);

/* ---- paged int8 KV cache ---------------------------------------------------- */

/* lh::paged_kv_append_q8 (src/kernels/kvcache_quant.hpp:41-46): one request;
 * k_new/v_new fp32 [n_kv_heads, seq_new, head_dim]; block_table device int32. */
LHB_API int lhb_paged_kv_append_q8(lhb_ctx* ctx, int8_t* k_pool, int8_t* v_pool, float* k_scales,
                                   float* v_scales, const float* k_new, const float* v_new,
                                   const int32_t* block_table, const lhb_paged_layout* layout,
                                   int past_len, int seq_new, void* stream);
/* Batched form of the same append for a decode step: request r appends
 * `seq_new` rows at position past_lens[r] (device array) through row r of
 * block_tables [n_requests, max_blocks_per_req]; k_new/v_new are
 * [n_requests, n_kv_heads, seq_new, head_dim].  The reference appends one
 * request per call (src/kernels/kvcache_quant.cpp:58-80); this is that loop
 * in one launch. */
LHB_API int lhb_paged_kv_append_q8_batched(lhb_ctx* ctx, int8_t* k_pool, int8_t* v_pool,
                                           float* k_scales, float* v_scales, const float* k_new,
                                           const float* v_new, const int32_t* block_tables,
                                           int max_blocks_per_req, const int32_t* past_lens,
                                           int n_requests, const lhb_paged_layout* layout,
                                           int seq_new, void* stream);
/* lh::paged_kv_append (src/kernels/kvcache.hpp:50-55): fp32 pools. */
LHB_API int lhb_paged_kv_append_f32(lhb_ctx* ctx, float* k_pool, float* v_pool,
                                    const float* k_new, const float* v_new,
                                    const int32_t* block_table, const lhb_paged_layout* layout,
                                    int past_len, int seq_new, void* stream);

/* ---- paged attention ---------------------------------------------------------- */

/* lh::paged_attention_q8 (src/kernels/kvcache_quant.hpp:51-57): one request. */
LHB_API int lhb_paged_attention_q8(lhb_ctx* ctx, const float* Q, const int8_t* K_pool,
                                   const int8_t* V_pool, const float* K_scales,
                                   const float* V_scales, const int32_t* block_table, int seq_len,
                                   float* O, const lhb_paged_attn_cfg* cfg,
                                   const lhb_paged_layout* layout, void* stream);
/* Batched int8 paged attention with the calling convention of
 * lh::paged_attention_batched (src/kernels/paged_attention.hpp:50-63) plus the
 * two scale pools: Q/O [n_requests, n_q_heads, seq_q, head_dim], block_tables
 * int32 [n_requests, max_blocks_per_req] (padding value ignored), seq_lens
 * int32 [n_requests], all in device memory. */
LHB_API int lhb_paged_attention_q8_batched(lhb_ctx* ctx, const float* Q, const int8_t* K_pool,
                                           const int8_t* V_pool, const float* K_scales,
                                           const float* V_scales, const int32_t* block_tables,
                                           int max_blocks_per_req, const int32_t* seq_lens,
                                           int n_requests, float* O,
                                           const lhb_paged_attn_cfg* cfg,
                                           const lhb_paged_layout* layout, void* stream);
/* No counterpart in the reference.  The same batched int8 decode attention as
 * lhb_paged_attention_q8_batched for callers that cannot let this library
 * allocate device memory and therefore have no context: a process that has
 * already committed all of HBM to its own pools, a plugin host that forbids
 * allocation after start-up, a loop that cannot tolerate the device-wide
 * synchronisation an allocation may cause.  The kernel's scratch (split-KV
 * partials, arrival counters, status word) lives in fixed arrays inside the
 * library image (about 8 MiB per GPU that loads the library, held until the
 * process exits); the call itself performs no cudaMalloc/cudaFree.
 * Limits: decode shape only (seq_q 1, head_dim 128, block_size 16, at most 4
 * query heads per KV head; otherwise LHB_ERR_UNSUPPORTED);
 * n_requests * n_kv_heads <= 4096 and split partials <= 8 MiB, otherwise
 * LHB_ERR_SCRATCH with a message in lhb_last_error().  The first call on a
 * device looks the arrays' device addresses up and sets a kernel attribute;
 * make that first call before any stream capture.  All calls on a device share
 * the arrays: calls that overlap on the GPU (different streams) race and must
 * be serialised by the caller. */
LHB_API int lhb_paged_attention_q8_batched_noalloc(const float* Q, const int8_t* K_pool,
                                                   const int8_t* V_pool, const float* K_scales,
                                                   const float* V_scales,
                                                   const int32_t* block_tables,
                                                   int max_blocks_per_req, const int32_t* seq_lens,
                                                   int n_requests, float* O,
                                                   const lhb_paged_attn_cfg* cfg,
                                                   const lhb_paged_layout* layout, void* stream);
/* lh::paged_attention / lh::paged_attention_batched on fp32 pools
 * (src/kernels/paged_attention.hpp:42-63). */
LHB_API int lhb_paged_attention_f32_batched(lhb_ctx* ctx, const float* Q, const float* K_pool,
                                            const float* V_pool, const int32_t* block_tables,
                                            int max_blocks_per_req, const int32_t* seq_lens,
                                            int n_requests, float* O,
                                            const lhb_paged_attn_cfg* cfg,
                                            const lhb_paged_layout* layout, void* stream);

/* ---- decode-step glue between the quantised GEMMs -------------------------------- */

/* lh::rmsnorm (src/kernels/normalization.hpp:21): y[r, :] = x[r, :] / rms(x[r, :]) * gamma. */
LHB_API int lhb_rmsnorm(lhb_ctx* ctx, const float* x, const float* gamma, float* y, int rows,
                        int dim, float eps, void* stream);
/* lh::rope (src/kernels/rope.hpp:19-21), in place on x = [seq, n_heads, head_dim]; row s sits
 * at position pos_offset + s.  interleaved != 0 rotates pairs (2i, 2i+1), else (i, i + d/2). */
LHB_API int lhb_rope(lhb_ctx* ctx, float* x, int seq, int n_heads, int head_dim, float theta_base,
                     float freq_scale, int interleaved, int pos_offset, void* stream);
/* The same rotation for a decode batch: x = [n_requests, n_heads, head_dim], one token per
 * request at positions[r] (a device array, e.g. the cache manager's seq_lens before the
 * append).  Equals lh::rope(x_r, 1, ..., pos_offset = positions[r]) for every request. */
LHB_API int lhb_rope_decode_batched(lhb_ctx* ctx, float* x, const int32_t* positions,
                                    int n_requests, int n_heads, int head_dim, float theta_base,
                                    float freq_scale, int interleaved, void* stream);
/* lh::swiglu (src/kernels/activation.hpp:34): x = [rows, 2*dim] (gate || value),
 * y[r, i] = gate * sigmoid(gate) * value. */
LHB_API int lhb_swiglu(lhb_ctx* ctx, const float* x, float* y, int rows, int dim, void* stream);

/* lhb_gemm_w4a16_groupwise with an operator of the decode step applied to the activations on the way
 * in (no counterpart in the reference; equals the two calls one after the other up to the order of the
 * sum of squares): prologue 1 = lh::rmsnorm(X [M, K], gamma [K], eps), 2 = lh::swiglu(X [M, 2K]).  The
 * normalised / activated tensor is never written.  Served for shapes of the tensor-core kernel whose
 * last slab of 16 rows has more than two rows; otherwise LHB_ERR_UNSUPPORTED, and the caller makes the
 * two calls. */
LHB_API int lhb_gemm_w4a16_groupwise_prologue(lhb_ctx* ctx, const float* X, int prologue,
                                              const float* gamma, float eps, const uint8_t* B_packed,
                                              const float* B_scales, float* C, int M, int N, int K,
                                              int group_size, float alpha, float beta, void* stream);

/* Decode-step fusion (no counterpart in the reference): qkv = [n_requests rows, row_stride floats
 * apart], each row = [n_q_heads | n_kv_heads | n_kv_heads] heads of head_dim, the output of a fused
 * QKV projection.  Equals lhb_rope_decode_batched on the q and on the k heads followed by
 * lhb_paged_kv_append_q8_batched(seq_new = 1) with the rotated k and the v heads, bit for bit:
 * rotated q goes to q_out [n_requests, n_q_heads, head_dim], k and v rows into the pools at
 * position positions[r] of request r. */
LHB_API int lhb_qkv_rope_append_q8_decode(lhb_ctx* ctx, const float* qkv, int64_t row_stride, float* q_out,
                                          int8_t* k_pool, int8_t* v_pool, float* k_scales,
                                          float* v_scales, const int32_t* block_tables,
                                          int max_blocks_per_req, const int32_t* positions,
                                          int n_requests, int n_q_heads,
                                          const lhb_paged_layout* layout, float theta_base,
                                          float freq_scale, int interleaved, void* stream);

/* ---- FP8 E4M3 ------------------------------------------------------------------------ */

/* lh::fp8_quantize_per_tensor / per_row / per_col (src/kernels/quant.hpp:81-94): E4M3 bytes
 * (src/kernels/dtypes.hpp:111-159: RNE, saturating at +-448, NaN/inf -> 0x7f) and fp32 scales
 * max|x| / 448 (1 if 0); one scale, one per row, one per column.  `scale_out` / `scales_out` are
 * device pointers.  Bit-exact with the reference. */
LHB_API int lhb_fp8_quantize_per_tensor(lhb_ctx* ctx, const float* src, uint8_t* dst, float* scale_out,
                                        int64_t n, void* stream);
LHB_API int lhb_fp8_quantize_per_row(lhb_ctx* ctx, const float* src, uint8_t* dst, float* scales_out,
                                     int rows, int dim, void* stream);
LHB_API int lhb_fp8_quantize_per_col(lhb_ctx* ctx, const float* src, uint8_t* dst, float* scales_out,
                                     int rows, int cols, void* stream);
/* lh::fp8_dequantize_per_tensor / per_row / per_col: dst = float(q) * scale; `mode` 0 = scales[0],
 * 1 = scales[row], 2 = scales[col] (device array). */
LHB_API int lhb_fp8_dequantize(lhb_ctx* ctx, const uint8_t* src, const float* scales, float* dst,
                               int rows, int cols, int mode, void* stream);
/* lh::gemm_fp8_e4m3 (src/kernels/gemm_quant.hpp:66-69): A [M, K] and B [K, N] E4M3 bytes, per-tensor
 * scales by value, C = beta*C + (alpha * A_scale * B_scale) * sum_k a*b with fp32 accumulation.
 * Shapes of lhb_gemm_w8a8_fast_path run on tcgen05 (kind::f8f6f4). */
LHB_API int lhb_gemm_fp8_e4m3(lhb_ctx* ctx, const uint8_t* A, const uint8_t* B, float A_scale,
                              float B_scale, float* C, int M, int N, int K, float alpha, float beta,
                              void* stream);
LHB_API int lhb_gemm_fp8_fast_path(int M, int N, int K);

/* ---- asymmetric int4 (extension; no counterpart in the reference) ------------------ */

/* The reference's int4 is symmetric with fp32 scales (src/kernels/quant.hpp:52-57).  This
 * variant keeps its packing - uint8 [K/2, N], low nibble = even k - with unsigned nibbles and
 * an fp16 scale and fp16 integer-valued zero-point per (group, column), both [K/G, N]:
 * lo = min(0, min w), hi = max(0, max w), s = fp16((hi - lo) / 15) (1 if 0),
 * z = clamp(rint(-lo / s), 0, 15), u = clamp(rint(w / s) + z, 0, 15), w' = (u - z) * s. */
LHB_API int lhb_q4a_quantize_groupwise(lhb_ctx* ctx, const float* src, uint8_t* packed,
                                       uint16_t* scales_f16, uint16_t* zeros_f16, int K, int N,
                                       int group_size, void* stream);
LHB_API int lhb_q4a_dequantize_groupwise(lhb_ctx* ctx, const uint8_t* packed,
                                         const uint16_t* scales_f16, const uint16_t* zeros_f16,
                                         float* dst, int K, int N, int group_size, void* stream);
/* C = beta*C + alpha * A @ dequant(B), the asymmetric counterpart of
 * lh::gemm_w4a16_groupwise (src/kernels/gemm_quant.hpp:54-57). */
LHB_API int lhb_gemm_w4a16_asym(lhb_ctx* ctx, const float* A, const uint8_t* B_packed,
                                const uint16_t* scales_f16, const uint16_t* zeros_f16, float* C,
                                int M, int N, int K, int group_size, float alpha, float beta,
                                void* stream);
/* 1 when the tensor-core decode kernel serves this shape. */
LHB_API int lhb_gemm_w4a16_asym_fast_path(int M, int N, int K, int group_size);

/* ---- device-resident cache manager ---------------------------------------------- */

/* Host bookkeeping of lh::CacheManager (src/runtime/cache_manager.hpp:34-110:
 * LIFO free list popping ascending ids, refcounts, all-or-nothing
 * ensure_capacity) with the storage moved to the GPU: int8 K/V pools + fp32
 * scale pools in the layout above, and the batched block tables
 * int32 [max_requests, max_blocks_per_req] (padded with -1) and seq_lens
 * int32 [max_requests] of lh::Scheduler::prepare_step
 * (src/runtime/scheduler.cpp:41-58) kept in device memory and patched
 * incrementally (row = request id) instead of rebuilt every step.  With
 * ctx == NULL the manager is "detached": the same bookkeeping with no device
 * storage (every device pointer getter returns NULL). */
typedef struct lhb_cache_manager lhb_cache_manager;

LHB_API int lhb_cm_create(lhb_ctx* ctx, const lhb_paged_layout* layout, int max_requests,
                          int max_blocks_per_req, lhb_cache_manager** out);
LHB_API int lhb_cm_destroy(lhb_cache_manager* cm);
LHB_API int lhb_cm_num_free_blocks(const lhb_cache_manager* cm);
LHB_API int lhb_cm_num_total_blocks(const lhb_cache_manager* cm);
/* Returns the new request id (dense, reused after release) or -1 when
 * max_requests are live. */
LHB_API int lhb_cm_create_request(lhb_cache_manager* cm);
LHB_API int lhb_cm_release_request(lhb_cache_manager* cm, int id, void* stream);
/* 1 on success, 0 on out-of-blocks (table unchanged), negative on error. */
LHB_API int lhb_cm_ensure_capacity(lhb_cache_manager* cm, int id, int seq_len, void* stream);
LHB_API int lhb_cm_set_seq_len(lhb_cache_manager* cm, int id, int seq_len, void* stream);
LHB_API int lhb_cm_reference_block(lhb_cache_manager* cm, int id, int logical_idx, int physical,
                                   void* stream);
LHB_API int lhb_cm_allocate_block(lhb_cache_manager* cm);
LHB_API int lhb_cm_release_block(lhb_cache_manager* cm, int physical);
LHB_API int lhb_cm_retain_block(lhb_cache_manager* cm, int physical);
LHB_API int lhb_cm_refcount(const lhb_cache_manager* cm, int physical);
LHB_API int lhb_cm_seq_len(const lhb_cache_manager* cm, int id);
/* Copies the host copy of request `id`'s block table into out[0..cap) and
 * returns its length. */
LHB_API int lhb_cm_block_table(const lhb_cache_manager* cm, int id, int32_t* out, int cap);
/* Device pointers (valid until lhb_cm_destroy). */
LHB_API int8_t* lhb_cm_k_pool(lhb_cache_manager* cm);
LHB_API int8_t* lhb_cm_v_pool(lhb_cache_manager* cm);
LHB_API float* lhb_cm_k_scales(lhb_cache_manager* cm);
LHB_API float* lhb_cm_v_scales(lhb_cache_manager* cm);
LHB_API int32_t* lhb_cm_block_tables(lhb_cache_manager* cm);
LHB_API int32_t* lhb_cm_seq_lens(lhb_cache_manager* cm);
LHB_API int lhb_cm_max_blocks_per_req(const lhb_cache_manager* cm);

/* ---- continuous-batching scheduler over the device cache manager ------------------- */

/* lh::Scheduler (src/runtime/scheduler.hpp:47-105): FIFO admission gated by max_concurrent and by an
 * all-or-nothing reservation of prompt + 1 tokens; commit_step counts one produced token per active
 * request, retires it on its flag or at max_new_tokens, else reserves the next slot.  Request bodies
 * are reduced to (prompt length, max_new_tokens): the scheduler never reads token values.
 * prepare_step returns the number of active requests, writes their ids (prepare order) to ids_out
 * when it is not NULL, and leaves the dense view of the reference's ActiveStep - block tables
 * [n_active, max_blocks_per_req] padded with -1 and seq_lens [n_active] - in device buffers
 * (lhb_sched_block_tables / lhb_sched_seq_lens), gathered on `stream` from the cache manager's
 * resident rows: only the active ids cross PCIe.  The view's width is the cache manager's fixed
 * max_blocks_per_req, not the step's maximum.  A scheduler over a detached cache manager keeps the
 * bookkeeping only. */
typedef struct lhb_scheduler lhb_scheduler;
LHB_API int lhb_sched_create(lhb_cache_manager* cm, int max_concurrent, lhb_scheduler** out);
LHB_API int lhb_sched_destroy(lhb_scheduler* s);
LHB_API int lhb_sched_submit(lhb_scheduler* s, int prompt_len, int max_new_tokens);   /* request id */
LHB_API int lhb_sched_has_work(const lhb_scheduler* s);
LHB_API int lhb_sched_queue_depth(const lhb_scheduler* s);
LHB_API int lhb_sched_active_size(const lhb_scheduler* s);
LHB_API double lhb_sched_last_step_occupancy(const lhb_scheduler* s);
LHB_API int lhb_sched_generated(const lhb_scheduler* s, int id);
LHB_API int lhb_sched_prepare_step(lhb_scheduler* s, int32_t* ids_out, int cap, void* stream);
LHB_API int lhb_sched_commit_step(lhb_scheduler* s, const uint8_t* completed, int n, void* stream);
LHB_API int32_t* lhb_sched_block_tables(lhb_scheduler* s);
LHB_API int32_t* lhb_sched_seq_lens(lhb_scheduler* s);
LHB_API int lhb_sched_max_blocks_per_req(const lhb_scheduler* s);

/* ---- exchange step of a tensor-parallel decode layer over NVLink peer memory ------- */

/* No reference interface stands behind these: the reference runs one model on one device
 * (src/runtime/scheduler.hpp:47).  They exist so that N processes, one per GPU, can run the decode
 * step with the projections sharded along N without a library collective between the GEMMs.
 *
 * lhb_peer_alloc returns zero-filled device memory that other processes on the same machine can map:
 * lhb_peer_export writes its 64-byte handle (send it to the peers by any means), lhb_peer_open maps a
 * peer's handle into this process with peer access enabled, lhb_peer_close / lhb_peer_free undo them
 * (close every mapping of a buffer before its owner frees it).
 *
 * lhb_peer_allgather_cols: this rank holds `local` [rows, width] fp32, columns
 * [rank*width, (rank+1)*width) of a row-major [rows, world*width] matrix that every rank needs.  One
 * launch stores the slab into its place in every rank's copy (dst_table[p] = base of rank p's copy as
 * mapped in this process, this rank's own pointer at p == rank; a DEVICE array of `world` pointers),
 * adds to rank p's arrival counters (flag_table[p] = rank p's uint32[world], peer-visible, zero at
 * start; a device array of `world` pointers) and returns once all ranks' slabs have arrived here.
 * `state` is this rank's own uint32[4], zero at start.  Rules: every rank issues the same sequence of
 * calls with the same shapes; width % 4 == 0 and 16-byte aligned buffers; consecutive calls target
 * different destination matrices, and a destination is not read between the call before it and the
 * call that fills it.  The wait is bounded by timeout_ms: after that the kernel records the silent
 * rank in `state` and returns; lhb_peer_status (synchronises `stream`) then gives LHB_ERR_TIMEOUT
 * and the data is not valid.  The launch can be captured in a CUDA graph. */
LHB_API int lhb_peer_alloc(void** out, size_t bytes);
/* The same service through the driver's virtual-memory-management calls, for buffers that kernels
 * stream into (the matrices of lhb_gemm_w8a8_sharded): lhb_peer_alloc_shareable creates zero-filled
 * device memory mapped with large pages, returns its address, the mapped size (`bytes` rounded up
 * to the allocation granularity) and a POSIX file descriptor for it; pass the descriptor to the
 * peer processes over a Unix socket (SCM_RIGHTS) and close it.  lhb_peer_open_fd maps a received
 * descriptor for the calling thread's current device; lhb_peer_unmap undoes either mapping (the
 * memory is freed when its owner and every peer have unmapped it and closed the descriptor).
 * Stores into these mappings run at the NVLink rate where stores into lhb_peer_open mappings of
 * several hundred megabytes did not (640 against 310 GB/s per GPU, four B200s).
 * LHB_ERR_UNSUPPORTED when the driver lacks the calls. */
LHB_API int lhb_peer_alloc_shareable(void** out, size_t bytes, int* fd_out, size_t* mapped_bytes);
LHB_API int lhb_peer_open_fd(int fd, size_t mapped_bytes, void** out);
LHB_API int lhb_peer_unmap(void* ptr, size_t mapped_bytes);
LHB_API int lhb_peer_free(void* ptr);
LHB_API int lhb_peer_export(void* ptr, unsigned char* handle64);
LHB_API int lhb_peer_open(const unsigned char* handle64, void** out);
LHB_API int lhb_peer_close(void* mapped);
LHB_API int lhb_peer_allgather_cols(const float* local, int rows, int width, void* const* dst_table,
                                    uint32_t* const* flag_table, uint32_t* state, int rank, int world,
                                    int timeout_ms, void* stream);
LHB_API int lhb_peer_status(const uint32_t* state, void* stream);
/* lhb_gemm_w4a16_groupwise (src/kernels/gemm_quant.hpp:54) on this rank's column shard of the weight, fused
 * with the exchange above: C [M, N] = alpha * A * dequant(B) + beta * C as usual, and the same values also
 * land in columns [rank*N, (rank+1)*N) of every rank's row-major [M, world*N] matrix (dst_table), stored
 * by the GEMM's own epilogue over NVLink; every completed column tile raises the arrival counters, and a
 * one-CTA launch that follows waits (bounded) until all ranks' tiles have arrived.  Same tables, state and
 * rules as lhb_peer_allgather_cols, and it counts as one call of that sequence.  Served by the tensor-core
 * kernel only (9 rows or more, group a multiple of 128); otherwise LHB_ERR_UNSUPPORTED and the caller runs
 * the GEMM and lhb_peer_allgather_cols separately. */
LHB_API int lhb_gemm_w4a16_groupwise_peer(lhb_ctx* ctx, const float* A, const uint8_t* B_packed, const float* B_scales,
                                          float* C, int M, int N, int K, int group_size, float alpha, float beta,
                                          void* const* dst_table, uint32_t* const* flag_table, uint32_t* state,
                                          int rank, int world, int timeout_ms, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LHB200_H */

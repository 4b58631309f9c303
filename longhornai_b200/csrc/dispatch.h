// Internal launch functions shared between the kernel files and api.cu.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "lhb200.h"

namespace lhb {

// generic kernels (gemm_generic.cu, paged_attention_generic.cu)
int launch_w4a16_generic(const float* A, const uint8_t* Bp, const float* Bs, float* C, int M, int N,
                         int K, int G, float alpha, float beta, cudaStream_t st);
int launch_w8a16_generic(const float* A, const int8_t* Bq, const float* Bs, float* C, int M, int N,
                         int K, float alpha, float beta, cudaStream_t st);
int launch_w8a8_generic(const int8_t* Aq, const int8_t* Bq, const float* as, const float* bs,
                        float* C, int M, int N, int K, float alpha, float beta, cudaStream_t st);
int launch_paged_attention_generic(lhb_ctx* ctx, bool q8, const float* Q, const void* Kp,
                                   const void* Vp, const float* Ks, const float* Vs,
                                   const int32_t* tables, int max_blocks, const int32_t* seq_lens,
                                   int seq_len_scalar, int n_req, float* O,
                                   const lhb_paged_attn_cfg& cfg, const lhb_paged_layout& L,
                                   cudaStream_t st);

// tensor-core skinny GEMMs (gemv_mma.cu)
bool w4a16_fast_ok(int M, int N, int K, int G);
bool w8a16_fast_ok(int M, int N, int K);
int launch_w4a16_fast(lhb_ctx* ctx, const float* A, const uint8_t* Bp, const float* Bs, float* C,
                      int M, int N, int K, int G, float alpha, float beta, cudaStream_t st);
int launch_w8a16_fast(lhb_ctx* ctx, const float* A, const int8_t* Bq, const float* Bs, float* C,
                      int M, int N, int K, float alpha, float beta, cudaStream_t st);

// tcgen05 W8A8 (gemm_w8a8_tc.cu)
bool w8a8_fast_ok(int M, int N, int K);
int launch_w8a8_fast(lhb_ctx* ctx, const int8_t* Aq, const int8_t* Bq, const float* as,
                     const float* bs, float* C, int M, int N, int K, float alpha, float beta,
                     cudaStream_t st);

int launch_w8a8_sharded(lhb_ctx* ctx, const int8_t* Aq, const int8_t* Bq, const float* as, const float* bs,
                        float* const* dst, int n_dst, int M, int N, int K, int64_t ldc, int col0, float alpha,
                        cudaStream_t st);

// split-KV decode attention (paged_attention_decode.cu)
bool decode_fast_ok(const lhb_paged_attn_cfg& cfg, const lhb_paged_layout& L);
int launch_decode_fast(lhb_ctx* ctx, const float* Q, const int8_t* Kp, const int8_t* Vp,
                       const float* Ks, const float* Vs, const int32_t* tables, int max_blocks,
                       const int32_t* seq_lens, int n_req, float* O, const lhb_paged_attn_cfg& cfg,
                       const lhb_paged_layout& L, cudaStream_t st);

// W4A16 with a prologue on the activations (1 = RMSNorm with gamma/eps, 2 = SwiGLU of [gate || value] rows)
// tensor-core W4A16 for a few rows up to a few hundred (gemm_w4a16_tc.cu); prologue 0 = none,
// 1 = RMSNorm (gamma, eps), 2 = SwiGLU of [gate || value] rows.  w4a16_tc_min_rows: the row count
// from which it is preferred over the GEMV kernel (environment LHB_W4TC_MIN_M overrides).
bool w4a16_tc_ok(int M, int N, int K, int G);
int w4a16_tc_min_rows();
// `peer` (optional): the result also goes to columns [col0, col0 + N) of every rank's [M, ld] matrix and each
// completed column tile of each slab adds one arrival at every rank; *arrivals_out = arrivals per rank.
struct W4Peer {
    void* const* dst_table;          // device array of `world` matrix bases as mapped in this process
    uint32_t* const* flag_table;     // device array of `world` arrival-counter arrays
    int world, rank, ld, col0;
};
int launch_w4a16_tc(lhb_ctx* ctx, const float* A, const uint8_t* Bp, const float* Bs, float* C, int M, int N, int K,
                    int G, float alpha, float beta, cudaStream_t st, int prologue, const float* gamma, float eps,
                    const W4Peer* peer = nullptr, uint32_t* arrivals_out = nullptr);
// waits (bounded) until every rank's counter in this rank's arrival array has grown by `add` (peer_gather.cu)
int launch_peer_wait(uint32_t* const* flag_table, uint32_t* state, int rank, int world, uint32_t add,
                     int timeout_ms, cudaStream_t st);
int launch_w4a16_fast_prologue(lhb_ctx* ctx, const float* X, int prologue, const float* gamma, float eps,
                               const uint8_t* Bp, const float* Bs, float* C, int M, int N, int K, int G, float alpha,
                               float beta, cudaStream_t st);

// fp8 E4M3 GEMM: generic kernel in fp8.cu, tcgen05 path in gemm_w8a8_tc.cu (shapes of w8a8_fast_ok)
int launch_fp8_generic(const uint8_t* A, const uint8_t* B, float combined, float* C, int M, int N, int K, float beta,
                       cudaStream_t st);
int launch_fp8_fast(lhb_ctx* ctx, const uint8_t* A, const uint8_t* B, float combined, float* C, int M, int N, int K,
                    float beta, cudaStream_t st);

// asymmetric int4 (fp16 scale and zero-point per group): generic kernel in quant_asym.cu,
// decode fast path in gemv_mma.cu
int launch_w4a16_asym_generic(const float* A, const uint8_t* Bp, const uint16_t* Bs, const uint16_t* Bz, float* C,
                              int M, int N, int K, int G, float alpha, float beta, cudaStream_t st);
bool w4a16_asym_fast_ok(int M, int N, int K, int G);
int launch_w4a16_asym_fast(lhb_ctx* ctx, const float* A, const uint8_t* Bp, const uint16_t* Bs, const uint16_t* Bz,
                           float* C, int M, int N, int K, int G, float alpha, float beta, cudaStream_t st);

// TMA tensor maps (tensor_map.cu): 2-D uint8 tensor [rows, cols] (cols
// contiguous, row pitch in bytes), box [box_rows, box_cols], 128-byte swizzle
// when swizzle128 is set.  Cached per context.
struct TensorMap;
int get_tensor_map_2d_u8(lhb_ctx* ctx, const void* base, uint64_t rows, uint64_t cols,
                         uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols,
                         bool swizzle128, TensorMap* out);
// the same for an fp32 tensor (cols and box_cols in elements), no swizzle
int get_tensor_map_2d_f32(lhb_ctx* ctx, const void* base, uint64_t rows, uint64_t cols,
                          uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols, TensorMap* out);
// fp32 with the 128-byte swizzle (box_cols * 4 == 128): the target of bulk stores from swizzled staging tiles
int get_tensor_map_2d_f32_sw128(lhb_ctx* ctx, const void* base, uint64_t rows, uint64_t cols,
                                uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols, TensorMap* out);
// and for an fp16 tensor
int get_tensor_map_2d_f16(lhb_ctx* ctx, const void* base, uint64_t rows, uint64_t cols,
                          uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols, TensorMap* out);

}  // namespace lhb

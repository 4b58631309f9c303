// W8A8 GEMM on the 5th-generation tensor cores: int8 x int8 -> int32 in TMEM,
// fp32 rescale in the epilogue.
//
// Operand layouts are the reference's (src/kernels/gemm_quant.hpp:35-45):
// A_q int8 [M, K] with K contiguous, B_q int8 [K, N] with N contiguous, i.e. B
// is "MN-major" for the tensor core.  Both are consumed as they lie: TMA brings
// 128-byte-swizzled tiles into shared memory and the tcgen05 shared-memory
// descriptors describe A as K-major and B as MN-major, so there is no weight
// transpose.
//
// One persistent CTA per SM walks 128 x 256 output tiles (M fastest, so the CTAs
// running together share A/B panels in L2).  Warp roles:
//   warp 0   TMA producer   4-stage ring, 48 KiB per stage (A 128x128, B 128x256)
//   warp 1   MMA issuer     one thread issues 4 tcgen05.mma (K = 32 each) per stage
//                           and commits the stage's "empty" barrier
//   warp 2   TMEM allocator 512 columns = two 128 x 256 int32 accumulators, so the
//                           epilogue of tile i overlaps the main loop of tile i+1
//   warps 4-7 epilogue      tcgen05.ld 32 lanes x 32 columns, then
//                           C = beta*C + ((alpha*a_s[m])*b_s[n])*float(acc)
// The int32 sums are exact and the epilogue multiplies in the reference's order
// with single roundings (src/kernels/gemm_quant.cpp:44-46), so the output is
// bit-identical to the reference.
//
// For M >= 256 the CTA-pair variant further down is used instead (two CTAs of a
// cluster share a 256 x 256 tile; LHB_W8A8_PAIR=0 forces this kernel).
//
// Every wait is bounded (ptx::mbar_wait); a timeout sets the context's status
// word, all roles fall through to the common exit and TMEM is freed.
#include <algorithm>
#include <cstdlib>

#include "common.cuh"
#include "dispatch.h"
#include "ptx.cuh"

namespace lhb {

constexpr int W8_BM = 128, W8_BN = 256, W8_BK = 128;
constexpr int W8_STAGES = 4;
constexpr int W8_A_BYTES = W8_BM * W8_BK;            // 16 KiB
constexpr int W8_B_BYTES = W8_BK * W8_BN;            // 32 KiB, two 128-column boxes
constexpr int W8_STAGE_BYTES = W8_A_BYTES + W8_B_BYTES;
constexpr int W8_THREADS = 256;
constexpr int W8_TMEM_COLS = 512;
// per epilogue warp: two 32 x 32 fp32 chunks on their way to peer memory (one being filled while the
// bulk stores of the other are still reading it); 1 KiB aligned for the 128-byte TMA swizzle
constexpr int W8_OUT_STAGE = 4 * 2 * 4096;
constexpr size_t W8_SMEM = 1024 + static_cast<size_t>(W8_STAGES) * W8_STAGE_BYTES + 256 + W8_OUT_STAGE;

// instruction descriptor: D = s32 (bits 4-5 = 2), A = B = signed int8 (bits 7-9,
// 10-12 = 1), A K-major (bit 15 = 0), B MN-major (bit 16 = 1), N >> 3 at bit 17,
// M >> 4 at bit 24
constexpr uint32_t W8_IDESC = (2u << 4) | (1u << 7) | (1u << 10) | (1u << 16) |
                              (static_cast<uint32_t>(W8_BN >> 3) << 17) |
                              (static_cast<uint32_t>(W8_BM >> 4) << 24);

constexpr int W8_MAX_DST = 8;

struct W8Params {
    const float* a_scales;
    const float* b_scales;
    float* C;              // == dst[0]
    // The result tile goes to n_dst matrices (row pitch ldc, first column col0): one for a plain call;
    // for the N-sharded call the same place in every rank's full-width matrix, dst[1..] being peer
    // memory written with plain stores from the epilogue while the main loop runs on.
    float* dst[W8_MAX_DST];
    int n_dst;
    int push_tma;          // 1: peer copies leave as TMA bulk stores (one per destination per chunk), 0: as plain stores
    int64_t ldc;
    int col0;
    int M, N, K;
    float alpha, beta;
    int tiles_m, tiles_n;
    int* status;
    float combined;        // fp8: alpha * A_scale * B_scale (a_scales / b_scales unused)
};

// Tensor maps of dst[1..] (fp32 [M, ldc], boxes of 32 rows x 32 columns, 128-byte swizzle) for the
// bulk-store form of the peer push; unused by a plain call.
struct W8DstMaps {
    TensorMap m[W8_MAX_DST - 1];
};

// fp8 (E4M3 x E4M3 -> fp32): same tiles, barriers and shared-memory descriptors; the
// instruction descriptor names D = f32 (bits 4-5 = 1) and A = B = E4M3 (formats 0)
constexpr uint32_t f8_idesc(int m, int n) {
    return (1u << 4) | (1u << 16) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// One 32-column chunk of one output row of the fp8 GEMM: C = beta*C + combined * acc, with the
// reference's separate roundings (src/kernels/gemm_quant.cpp:87-104).
__device__ __forceinline__ void f8_store_chunk(int64_t row_off, int nb, const uint32_t (&r)[32], const W8Params& p) {
    float* crow = p.C + row_off;
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
        if (nb + j >= p.N) break;                      // N % 16 == 0: whole float4 in range
        float4 v;
        v.x = __fmul_rn(p.combined, __uint_as_float(r[j]));
        v.y = __fmul_rn(p.combined, __uint_as_float(r[j + 1]));
        v.z = __fmul_rn(p.combined, __uint_as_float(r[j + 2]));
        v.w = __fmul_rn(p.combined, __uint_as_float(r[j + 3]));
        float4* dst = reinterpret_cast<float4*>(crow + nb + j);
        if (p.beta != 0.0f) {
            const float4 o = *dst;
            if (p.beta == 1.0f) {
                v.x = __fadd_rn(o.x, v.x); v.y = __fadd_rn(o.y, v.y); v.z = __fadd_rn(o.z, v.z); v.w = __fadd_rn(o.w, v.w);
            } else {
                v.x = __fadd_rn(__fmul_rn(o.x, p.beta), v.x); v.y = __fadd_rn(__fmul_rn(o.y, p.beta), v.y);
                v.z = __fadd_rn(__fmul_rn(o.z, p.beta), v.z); v.w = __fadd_rn(__fmul_rn(o.w, p.beta), v.w);
            }
        }
        *dst = v;
    }
}


// Tile index -> (row block, column block).  Row blocks run fastest for a plain call (consecutive
// CTAs share a weight tile in L2).  The N-sharded call runs column blocks fastest: its epilogues
// store into every rank's matrix, and the tiles in flight then touch a band of rows - a few
// hundred pages of each peer mapping - instead of every row of every matrix, which is more pages
// than the translation caches hold when the peer mappings have small pages (cudaIpc mappings,
// 8192 x 28672 fp32 on 4 GPUs: 9.2 ms row-fastest, 2.3 ms column-fastest; large-page mappings: 1.1 ms).
__device__ __forceinline__ void w8_tile_blocks(int tile, int tiles_m, int tiles_n, bool n_fastest, int& mb, int& nb) {
    if (n_fastest) { mb = tile / tiles_n; nb = tile - mb * tiles_n; }
    else { nb = tile / tiles_m; mb = tile - nb * tiles_m; }
}

// The same chunk for the other ranks of an N-sharded call: a warp holds 32 rows x 32 columns, one row
// per lane.  Stored as they are, every 16-byte piece of a lane would cross NVLink as a request of
// its own; staged through 4 KiB of shared memory (XOR-swizzled against bank conflicts) the warp
// writes whole 128-byte row pieces, four rows per instruction.  Rows >= M are not written.
__device__ __forceinline__ void w8_push_chunk(float4* stg, int lane, int row0, int nb, const uint32_t (&r)[32], float sa,
                                              const W8Params& p) {
#pragma unroll
    for (int j4 = 0; j4 < 8; ++j4) {
        const float4 bs = __ldg(reinterpret_cast<const float4*>(p.b_scales + nb + 4 * j4));
        float4 v;
        v.x = __fmul_rn(__fmul_rn(sa, bs.x), static_cast<float>(static_cast<int>(r[4 * j4])));
        v.y = __fmul_rn(__fmul_rn(sa, bs.y), static_cast<float>(static_cast<int>(r[4 * j4 + 1])));
        v.z = __fmul_rn(__fmul_rn(sa, bs.z), static_cast<float>(static_cast<int>(r[4 * j4 + 2])));
        v.w = __fmul_rn(__fmul_rn(sa, bs.w), static_cast<float>(static_cast<int>(r[4 * j4 + 3])));
        stg[lane * 8 + (j4 ^ (lane & 7))] = v;
    }
    __syncwarp();
#pragma unroll
    for (int it = 0; it < 8; ++it) {
        const int idx = it * 32 + lane, rr = idx >> 3, j4 = idx & 7;
        const float4 v = stg[rr * 8 + (j4 ^ (rr & 7))];
        if (row0 + rr < p.M) {
            const int64_t off = static_cast<int64_t>(row0 + rr) * p.ldc + p.col0 + nb + 4 * j4;
            for (int d = 1; d < p.n_dst; ++d) *reinterpret_cast<float4*>(p.dst[d] + off) = v;
        }
    }
    __syncwarp();                                         // the tile is free for the next chunk
}

// The bulk-store form of the same push: the staged chunk (the XOR pattern above is exactly the TMA
// 128-byte swizzle) leaves as one cp.async.bulk.tensor store per destination, issued by lane 0.  The
// copy engine of the SM then feeds NVLink with whole rows of the box and the warp goes back to the
// accumulator at once; `use` alternates between the warp's two staging tiles, and a tile is refilled
// only after the stores issued from it two chunks earlier have read it.  Rows >= M are clipped by
// the tensor map.
__device__ __forceinline__ void w8_push_chunk_tma(float4* stg2, int use, int lane, int row0, int nb, const uint32_t (&r)[32],
                                                  float sa, const W8Params& p, const W8DstMaps& maps) {
    float4* stg = stg2 + (use & 1) * 256;
    if (lane == 0) ptx::bulk_wait_group_read<1>();
    __syncwarp();
#pragma unroll
    for (int j4 = 0; j4 < 8; ++j4) {
        const float4 bs = __ldg(reinterpret_cast<const float4*>(p.b_scales + nb + 4 * j4));
        float4 v;
        v.x = __fmul_rn(__fmul_rn(sa, bs.x), static_cast<float>(static_cast<int>(r[4 * j4])));
        v.y = __fmul_rn(__fmul_rn(sa, bs.y), static_cast<float>(static_cast<int>(r[4 * j4 + 1])));
        v.z = __fmul_rn(__fmul_rn(sa, bs.z), static_cast<float>(static_cast<int>(r[4 * j4 + 2])));
        v.w = __fmul_rn(__fmul_rn(sa, bs.w), static_cast<float>(static_cast<int>(r[4 * j4 + 3])));
        stg[lane * 8 + (j4 ^ (lane & 7))] = v;
    }
    ptx::fence_proxy_async_shared();                      // the bulk copy reads what this thread just wrote
    __syncwarp();
    if (lane == 0 && row0 < p.M) {
        const uint32_t src = ptx::smem_u32(stg);
        for (int d = 1; d < p.n_dst; ++d) ptx::tma_store_2d(&maps.m[d - 1], src, p.col0 + nb, row0);
    }
    if (lane == 0) ptx::bulk_commit_group();
}

// One 32-column chunk of one output row: C = beta*C + ((alpha*a_s)*b_s[n])*float(acc),
// multiplied in the reference's order with single roundings.
__device__ __forceinline__ void w8_store_chunk(int64_t row_off, int nb, const uint32_t (&r)[32], float sa,
                                               const W8Params& p) {
    float* crow = p.C + row_off;
    if (nb + 32 <= p.N) {
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
            const float4 bs = __ldg(reinterpret_cast<const float4*>(p.b_scales + nb + j));
            float4 v;
            v.x = __fmul_rn(__fmul_rn(sa, bs.x), static_cast<float>(static_cast<int>(r[j])));
            v.y = __fmul_rn(__fmul_rn(sa, bs.y), static_cast<float>(static_cast<int>(r[j + 1])));
            v.z = __fmul_rn(__fmul_rn(sa, bs.z), static_cast<float>(static_cast<int>(r[j + 2])));
            v.w = __fmul_rn(__fmul_rn(sa, bs.w), static_cast<float>(static_cast<int>(r[j + 3])));
            float4* dst = reinterpret_cast<float4*>(crow + nb + j);
            if (p.beta != 0.0f) {
                const float4 o = *dst;
                if (p.beta == 1.0f) {
                    v.x = __fadd_rn(o.x, v.x); v.y = __fadd_rn(o.y, v.y);
                    v.z = __fadd_rn(o.z, v.z); v.w = __fadd_rn(o.w, v.w);
                } else {
                    v.x = __fadd_rn(__fmul_rn(o.x, p.beta), v.x); v.y = __fadd_rn(__fmul_rn(o.y, p.beta), v.y);
                    v.z = __fadd_rn(__fmul_rn(o.z, p.beta), v.z); v.w = __fadd_rn(__fmul_rn(o.w, p.beta), v.w);
                }
            }
            *dst = v;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            if (nb + j < p.N) {
                float v = __fmul_rn(__fmul_rn(sa, p.b_scales[nb + j]), static_cast<float>(static_cast<int>(r[j])));
                float* dst = crow + nb + j;
                if (p.beta == 1.0f) v = __fadd_rn(*dst, v);
                else if (p.beta != 0.0f) v = __fadd_rn(__fmul_rn(*dst, p.beta), v);
                *dst = v;
            }
        }
    }
}

template <bool F8>
__global__ void __launch_bounds__(W8_THREADS, 1)
gemm_w8a8_tc_kernel(const __grid_constant__ TensorMap tmA, const __grid_constant__ TensorMap tmB,
                    const W8Params p, const __grid_constant__ W8DstMaps dmaps) {
    extern __shared__ uint8_t w8_smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(w8_smem_raw) + 1023) & ~uintptr_t(1023));
    float4* stage_out = reinterpret_cast<float4*>(smem + W8_STAGES * W8_STAGE_BYTES);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + W8_STAGES * W8_STAGE_BYTES + W8_OUT_STAGE);
    // bars[0..3] full, [4..7] empty, [8..9] tmem_full, [10..11] tmem_empty
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar0 = ptx::smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8 * s; };
    auto empty_bar = [&](int s) { return bar0 + 8 * (W8_STAGES + s); };
    auto tfull_bar = [&](int b) { return bar0 + 8 * (2 * W8_STAGES + b); };
    auto tempty_bar = [&](int b) { return bar0 + 8 * (2 * W8_STAGES + 2 + b); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < W8_STAGES; ++s) { ptx::mbar_init(full_bar(s), 1); ptx::mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < 2; ++b) { ptx::mbar_init(tfull_bar(b), 1); ptx::mbar_init(tempty_bar(b), 128); }
        *abort_flag = 0;
        ptx::fence_mbar_init();
        ptx::prefetch_tmap(&tmA);
        ptx::prefetch_tmap(&tmB);
    }
    if (warp == 2) {
        ptx::tmem_alloc(ptx::smem_u32(tmem_slot), W8_TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int n_tiles = p.tiles_m * p.tiles_n;
    const int num_kb = (p.K + W8_BK - 1) / W8_BK;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            for (int tile = blockIdx.x; tile < n_tiles && !*abort_flag; tile += gridDim.x) {
                int mb_, nb_;
                w8_tile_blocks(tile, p.tiles_m, p.tiles_n, p.n_dst > 1, mb_, nb_);
                const int m0 = mb_ * W8_BM, n0 = nb_ * W8_BN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % W8_STAGES;
                    if (!ptx::mbar_wait(empty_bar(s), ((it / W8_STAGES) & 1) ^ 1, abort_flag, p.status)) break;
                    ptx::mbar_expect_tx(full_bar(s), W8_STAGE_BYTES);
                    const uint32_t sa = ptx::smem_u32(smem + s * W8_STAGE_BYTES);
                    ptx::tma_load_2d(sa, &tmA, kb * W8_BK, m0, full_bar(s));
                    ptx::tma_load_2d(sa + W8_A_BYTES, &tmB, n0, kb * W8_BK, full_bar(s));
                    ptx::tma_load_2d(sa + W8_A_BYTES + W8_BK * 128, &tmB, n0 + 128, kb * W8_BK, full_bar(s));
                }
            }
            // drain: every stage this thread armed completes before the CTA may exit
            const int armed = it < W8_STAGES ? it : W8_STAGES;
            for (int j = 0; j < armed; ++j) {
                const int jt = it - 1 - j;
                const int s = jt % W8_STAGES;
                const uint64_t t0 = ptx::global_timer_ns();
                while (!ptx::mbar_try_wait(full_bar(s), (jt / W8_STAGES) & 1))
                    if (ptx::global_timer_ns() - t0 > 200000000ull) break;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int it = 0, ti = 0;
            for (int tile = blockIdx.x; tile < n_tiles && !*abort_flag; tile += gridDim.x, ++ti) {
                const int buf = ti & 1;
                if (!ptx::mbar_wait(tempty_bar(buf), ((ti >> 1) & 1) ^ 1, abort_flag, p.status)) break;
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * W8_BN;
                bool ok = true;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % W8_STAGES;
                    if (!ptx::mbar_wait(full_bar(s), (it / W8_STAGES) & 1, abort_flag, p.status)) { ok = false; break; }
                    ptx::tc_fence_after();
                    const uint32_t sa = ptx::smem_u32(smem + s * W8_STAGE_BYTES);
                    const uint32_t sb = sa + W8_A_BYTES;
#pragma unroll
                    for (int k4 = 0; k4 < W8_BK / 32; ++k4) {
                        // A: K-major, rows of 128 B, 8-row groups 1024 B apart; K advances 32 B inside the row
                        const uint64_t da = ptx::smem_desc_sw128(sa + k4 * 32, 16, 1024);
                        // B: MN-major, 128 columns per atom row, 8 k-rows = 1024 B, the second
                        // 128-column box lies W8_BK*128 bytes further; K advances 32 rows
                        const uint64_t db = ptx::smem_desc_sw128(sb + k4 * 32 * 128, W8_BK * 128, 1024);
                        if (F8) ptx::mma_f8_ss(d_tmem, da, db, f8_idesc(W8_BM, W8_BN), (kb | k4) != 0 ? 1u : 0u);
                        else ptx::mma_i8_ss(d_tmem, da, db, W8_IDESC, (kb | k4) != 0 ? 1u : 0u);
                    }
                    ptx::tc_commit(empty_bar(s));
                }
                if (!ok) break;
                ptx::tc_commit(tfull_bar(buf));
            }
        }
    } else if (warp >= 4) {
        const int q = warp - 4;                            // TMEM lane quarter this warp may read
        int ti = 0;
        int n_push = 0;
        for (int tile = blockIdx.x; tile < n_tiles && !*abort_flag; tile += gridDim.x, ++ti) {
            const int buf = ti & 1;
            int mb_, nb_;
            w8_tile_blocks(tile, p.tiles_m, p.tiles_n, p.n_dst > 1, mb_, nb_);
            const int m0 = mb_ * W8_BM, n0 = nb_ * W8_BN;
            if (!ptx::mbar_wait(tfull_bar(buf), (ti >> 1) & 1, abort_flag, p.status)) break;
            ptx::tc_fence_after();
            const int row = m0 + 32 * q + lane;
            const bool row_ok = row < p.M;
            const float sa = (row_ok && !F8) ? __fmul_rn(p.alpha, p.a_scales[row]) : 0.0f;
            const int64_t crow = static_cast<int64_t>(row_ok ? row : 0) * p.ldc + p.col0;
#pragma unroll 1
            for (int c = 0; c < W8_BN / 32; ++c) {
                uint32_t r[32];
                ptx::tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(32 * q) << 16) + buf * W8_BN + c * 32, r);
                ptx::tmem_ld_wait();
                if (c == W8_BN / 32 - 1) {                 // accumulator fully read: hand it back
                    ptx::tc_fence_before();
                    ptx::mbar_arrive(tempty_bar(buf));
                }
                const int nb = n0 + c * 32;
                if (nb >= p.N) continue;
                if (!F8 && p.n_dst > 1 && nb + 32 <= p.N) {    // warp-uniform: all 32 lanes take part
                    if (p.push_tma) w8_push_chunk_tma(stage_out + q * 512, n_push++, lane, row - lane, nb, r, sa, p, dmaps);
                    else w8_push_chunk(stage_out + q * 512, lane, row - lane, nb, r, sa, p);
                }
                if (!row_ok) continue;
                if (F8) f8_store_chunk(crow, nb, r, p);
                else w8_store_chunk(crow, nb, r, sa, p);
            }
        }
        if (lane == 0) ptx::bulk_wait_group<0>();          // this warp's bulk stores have left shared memory and landed
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 2) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, W8_TMEM_COLS);
    }
}


// ---------------------------------------------------------------------------
// CTA-pair variant: two CTAs of a cluster share one 256 x 256 output tile.
// Each CTA loads its 128 rows of A and its 128 columns of B (32 KiB per stage
// instead of 48), the leader issues tcgen05.mma.cta_group::2 (M = 256) that
// reads both CTAs' shared memory, and each CTA's TMEM receives its 128 rows.
// Shared-memory traffic per MMA drops by a third, which is what limits the
// single-CTA kernel.  Barriers: "full" lives in the leader (both CTAs' loads
// report there), "empty" and "accumulator full" exist in both CTAs (the leader
// commits to each), "accumulator empty" lives in the leader (256 arrivals).
// ---------------------------------------------------------------------------
constexpr int W8P_STAGES = 6;
constexpr int W8P_A_BYTES = 128 * W8_BK;             // this CTA's 128 rows
constexpr int W8P_B_BYTES = W8_BK * 128;             // this CTA's 128 columns
constexpr int W8P_STAGE_BYTES = W8P_A_BYTES + W8P_B_BYTES;
constexpr size_t W8P_SMEM = 1024 + static_cast<size_t>(W8P_STAGES) * W8P_STAGE_BYTES + 256 + W8_OUT_STAGE;
constexpr uint32_t W8P_IDESC = (2u << 4) | (1u << 7) | (1u << 10) | (1u << 16) |
                               (static_cast<uint32_t>(256 >> 3) << 17) | (static_cast<uint32_t>(256 >> 4) << 24);

template <bool F8>
__global__ void __launch_bounds__(W8_THREADS, 1)
gemm_w8a8_tc_pair_kernel(const __grid_constant__ TensorMap tmA, const __grid_constant__ TensorMap tmB,
                         const W8Params p, const __grid_constant__ W8DstMaps dmaps) {
    extern __shared__ uint8_t w8_smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(w8_smem_raw) + 1023) & ~uintptr_t(1023));
    float4* stage_out = reinterpret_cast<float4*>(smem + W8P_STAGES * W8P_STAGE_BYTES);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + W8P_STAGES * W8P_STAGE_BYTES + W8_OUT_STAGE);
    // bars[0..5] full, [6..11] empty, [12..13] tmem_full, [14..15] tmem_empty
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_ctarank();       // 0 = leader
    const uint32_t bar0 = ptx::smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8 * s; };
    auto empty_bar = [&](int s) { return bar0 + 8 * (W8P_STAGES + s); };
    auto tfull_bar = [&](int b) { return bar0 + 8 * (2 * W8P_STAGES + b); };
    auto tempty_bar = [&](int b) { return bar0 + 8 * (2 * W8P_STAGES + 2 + b); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < W8P_STAGES; ++s) { ptx::mbar_init(full_bar(s), 1); ptx::mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < 2; ++b) { ptx::mbar_init(tfull_bar(b), 1); ptx::mbar_init(tempty_bar(b), 256); }
        *abort_flag = 0;
        ptx::fence_mbar_init();
        ptx::prefetch_tmap(&tmA);
        ptx::prefetch_tmap(&tmB);
    }
    if (warp == 2) {
        ptx::tmem_alloc_pair(ptx::smem_u32(tmem_slot), W8_TMEM_COLS);
        ptx::tmem_relinquish_pair();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync_all();                            // both CTAs' barriers exist before anyone signals them
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int tiles_m = (p.M + 255) / 256;
    const int n_tiles = tiles_m * p.tiles_n;
    const int num_kb = (p.K + W8_BK - 1) / W8_BK;
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            for (int tile = pair; tile < n_tiles && !*abort_flag; tile += n_pairs) {
                int mb_, nb_;
                w8_tile_blocks(tile, tiles_m, p.tiles_n, p.n_dst > 1, mb_, nb_);
                const int m0 = mb_ * 256 + 128 * rank, n0 = nb_ * W8_BN + 128 * rank;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % W8P_STAGES;
                    if (!ptx::mbar_wait(empty_bar(s), ((it / W8P_STAGES) & 1) ^ 1, abort_flag, p.status)) break;
                    const uint32_t leader_full = ptx::mapa_shared(full_bar(s), 0);
                    if (rank == 0) ptx::mbar_expect_tx(full_bar(s), 2 * W8P_STAGE_BYTES);   // both CTAs' bytes
                    const uint32_t sa = ptx::smem_u32(smem + s * W8P_STAGE_BYTES);
                    ptx::tma_load_2d_pair(sa, &tmA, kb * W8_BK, m0, leader_full);
                    ptx::tma_load_2d_pair(sa + W8P_A_BYTES, &tmB, n0, kb * W8_BK, leader_full);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            int it = 0, ti = 0;
            for (int tile = pair; tile < n_tiles && !*abort_flag; tile += n_pairs, ++ti) {
                const int buf = ti & 1;
                if (!ptx::mbar_wait(tempty_bar(buf), ((ti >> 1) & 1) ^ 1, abort_flag, p.status)) break;
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * W8_BN;
                bool ok = true;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % W8P_STAGES;
                    if (!ptx::mbar_wait(full_bar(s), (it / W8P_STAGES) & 1, abort_flag, p.status)) { ok = false; break; }
                    ptx::tc_fence_after();
                    const uint32_t sa = ptx::smem_u32(smem + s * W8P_STAGE_BYTES);
                    const uint32_t sb = sa + W8P_A_BYTES;
#pragma unroll
                    for (int k4 = 0; k4 < W8_BK / 32; ++k4) {
                        const uint64_t da = ptx::smem_desc_sw128(sa + k4 * 32, 16, 1024);
                        const uint64_t db = ptx::smem_desc_sw128(sb + k4 * 32 * 128, 16, 1024);
                        if (F8) ptx::mma_f8_ss_pair(d_tmem, da, db, f8_idesc(256, 256), (kb | k4) != 0 ? 1u : 0u);
                        else ptx::mma_i8_ss_pair(d_tmem, da, db, W8P_IDESC, (kb | k4) != 0 ? 1u : 0u);
                    }
                    ptx::tc_commit_pair(ptx::mapa_shared(empty_bar(s), 0));     // stage free in both CTAs
                    ptx::tc_commit_pair(ptx::mapa_shared(empty_bar(s), 1));
                }
                if (!ok) break;
                ptx::tc_commit_pair(ptx::mapa_shared(tfull_bar(buf), 0));
                ptx::tc_commit_pair(ptx::mapa_shared(tfull_bar(buf), 1));
            }
        }
    } else if (warp >= 4) {
        const int q = warp - 4;
        int ti = 0, n_push = 0;
        for (int tile = pair; tile < n_tiles && !*abort_flag; tile += n_pairs, ++ti) {
            const int buf = ti & 1;
            int mb_, nb_;
            w8_tile_blocks(tile, tiles_m, p.tiles_n, p.n_dst > 1, mb_, nb_);
            const int m0 = mb_ * 256 + 128 * rank, n0 = nb_ * W8_BN;
            if (!ptx::mbar_wait(tfull_bar(buf), (ti >> 1) & 1, abort_flag, p.status)) break;
            ptx::tc_fence_after();
            const int row = m0 + 32 * q + lane;
            const bool row_ok = row < p.M;
            const float sa = (row_ok && !F8) ? __fmul_rn(p.alpha, p.a_scales[row]) : 0.0f;
            const int64_t crow = static_cast<int64_t>(row_ok ? row : 0) * p.ldc + p.col0;
            const uint32_t leader_tempty = ptx::mapa_shared(tempty_bar(buf), 0);
#pragma unroll 1
            for (int c = 0; c < W8_BN / 32; ++c) {
                uint32_t r[32];
                ptx::tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(32 * q) << 16) + buf * W8_BN + c * 32, r);
                ptx::tmem_ld_wait();
                if (c == W8_BN / 32 - 1) {
                    ptx::tc_fence_before();
                    ptx::mbar_arrive_cluster(leader_tempty);
                }
                const int nb = n0 + c * 32;
                if (nb >= p.N) continue;
                if (!F8 && p.n_dst > 1 && nb + 32 <= p.N) {    // warp-uniform: all 32 lanes take part
                    if (p.push_tma) w8_push_chunk_tma(stage_out + q * 512, n_push++, lane, row - lane, nb, r, sa, p, dmaps);
                    else w8_push_chunk(stage_out + q * 512, lane, row - lane, nb, r, sa, p);
                }
                if (!row_ok) continue;
                if (F8) f8_store_chunk(crow, nb, r, p);
                else w8_store_chunk(crow, nb, r, sa, p);
            }
        }
        if (lane == 0) ptx::bulk_wait_group<0>();          // this warp's bulk stores have left shared memory and landed
    }

    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync_all();                            // neither CTA frees memory the pair may still touch
    if (warp == 2) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc_pair(tmem_base, W8_TMEM_COLS);
    }
}

bool w8a8_fast_ok(int M, int N, int K) {
    return M >= 64 && N >= 128 && K >= 128 && (N % 16) == 0 && (K % 16) == 0;
}

template <bool F8>
static int launch_tc(lhb_ctx* ctx, const void* Aq, const void* Bq, W8Params p, cudaStream_t st) {
    const int M = p.M, N = p.N, K = p.K;
    TensorMap tmA, tmB;
    if (int e = get_tensor_map_2d_u8(ctx, Aq, M, K, K, W8_BM, W8_BK, true, &tmA)) return e;
    if (int e = get_tensor_map_2d_u8(ctx, Bq, K, N, N, W8_BK, 128, true, &tmB)) return e;
    static bool attr_set[64] = {};
    if (!attr_set[ctx->device & 63]) {
        LHB_CUDA(cudaFuncSetAttribute(gemm_w8a8_tc_kernel<F8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(W8_SMEM)));
        LHB_CUDA(cudaFuncSetAttribute(gemm_w8a8_tc_pair_kernel<F8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(W8P_SMEM)));
        attr_set[ctx->device & 63] = true;
    }
    p.tiles_m = ceil_div(M, W8_BM); p.tiles_n = ceil_div(N, W8_BN);
    p.status = ctx->status_word;
    if (p.n_dst == 0) {                                      // a plain call: one row-major [M, N] result
        p.n_dst = 1; p.dst[0] = p.C; p.ldc = N; p.col0 = 0;
    }
    static W8DstMaps no_maps = {};
    W8DstMaps pushed;
    const W8DstMaps* dmaps = &no_maps;
    if (p.n_dst > 1) {
        p.push_tma = knobs().w8a8_push_tma ? 1 : 0;
        if (p.push_tma) {
            for (int d = 1; d < p.n_dst; ++d)
                if (int e = get_tensor_map_2d_f32_sw128(ctx, p.dst[d], M, p.ldc, p.ldc * 4, 32, 32, &pushed.m[d - 1])) return e;
            for (int d = p.n_dst; d < W8_MAX_DST; ++d) pushed.m[d - 1] = pushed.m[0];
            dmaps = &pushed;
        }
    }
    const bool use_pair = knobs().w8a8_pair;
    // a caller that overlaps its own communication kernels keeps some SMs out of the persistent grid
    const int sms = ctx->sm_limit > 0 ? std::min(ctx->sm_count, ctx->sm_limit) : ctx->sm_count;
    if (use_pair && M >= 256) {
        const int tiles = ceil_div(M, 256) * p.tiles_n;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * std::max(1, std::min(sms / 2, tiles)), 1, 1);   // at least one pair, whatever the SM limit
        cfg.blockDim = dim3(W8_THREADS, 1, 1);
        cfg.dynamicSmemBytes = W8P_SMEM;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        LHB_CUDA(cudaLaunchKernelEx(&cfg, gemm_w8a8_tc_pair_kernel<F8>, tmA, tmB, p, *dmaps));
        return LHB_OK;
    }
    const int grid = std::min(sms, p.tiles_m * p.tiles_n);
    gemm_w8a8_tc_kernel<F8><<<grid, W8_THREADS, W8_SMEM, st>>>(tmA, tmB, p, *dmaps);
    LHB_LAUNCH_CHECK();
    return LHB_OK;
}

int launch_w8a8_fast(lhb_ctx* ctx, const int8_t* Aq, const int8_t* Bq, const float* as,
                     const float* bs, float* C, int M, int N, int K, float alpha, float beta,
                     cudaStream_t st) {
    W8Params p{};
    p.a_scales = as; p.b_scales = bs; p.C = C; p.M = M; p.N = N; p.K = K;
    p.alpha = alpha; p.beta = beta;
    return launch_tc<false>(ctx, Aq, Bq, p, st);
}

// N-sharded form: the [M, N] result of this rank's weight slab lands in columns [col0, col0 + N) of the
// [M, ldc] matrix of every rank (dst[0] this rank's own, the others peer memory).
int launch_w8a8_sharded(lhb_ctx* ctx, const int8_t* Aq, const int8_t* Bq, const float* as, const float* bs,
                        float* const* dst, int n_dst, int M, int N, int K, int64_t ldc, int col0, float alpha,
                        cudaStream_t st) {
    if (n_dst < 1 || n_dst > W8_MAX_DST) return LHB_ERR_BAD_SHAPE;
    W8Params p{};
    p.a_scales = as; p.b_scales = bs; p.C = dst[0]; p.M = M; p.N = N; p.K = K;
    p.alpha = alpha; p.beta = 0.0f;
    for (int d = 0; d < n_dst; ++d) p.dst[d] = dst[d];
    p.n_dst = n_dst; p.ldc = ldc; p.col0 = col0;
    return launch_tc<false>(ctx, Aq, Bq, p, st);
}

// fp8 E4M3 GEMM with per-tensor scales folded into `combined` (same shapes as the int8 kernel)
int launch_fp8_fast(lhb_ctx* ctx, const uint8_t* A, const uint8_t* B, float combined, float* C, int M, int N, int K,
                    float beta, cudaStream_t st) {
    W8Params p{};
    p.C = C; p.M = M; p.N = N; p.K = K;
    p.alpha = 1.0f; p.beta = beta; p.combined = combined;
    return launch_tc<true>(ctx, A, B, p, st);
}

}  // namespace lhb

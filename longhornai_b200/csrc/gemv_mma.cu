// Skinny weight-only GEMMs (decode GEMV, M <= 16 per launch) for int4-group
// and int8-per-channel weights in the reference's own layouts:
//   W4: packed uint8 [K/2, N], byte (k/2, n), low nibble = even k
//       (src/kernels/quant.hpp:52-57), fp32 scales [K/G, N];
//   W8: int8 [K, N], fp32 scales [N] (src/kernels/quant.hpp:45-48).
// Both layouts are N-contiguous, i.e. the reduction axis is the slow axis.
//
// The path is HBM-bound: the weight bytes are read exactly once, so the kernel
// is built to spend as few issue slots per weight as possible.
//
//   TMA (2-D, 128-byte swizzle)  global -> shared, two 64-row x 128-column boxes
//       per stage (a CTA owns 256 columns), 3-deep ring, all of it in flight at once;
//   ldmatrix.trans on the raw bytes: one 8x8 b16 matrix = 8 byte-rows x 16
//       columns; the transposed fragment hands every thread the bytes of two
//       adjacent columns at two consecutive rows;
//   int4 -> int8 without arithmetic: a nibble moved to the top of its byte IS
//       the two's-complement int8 value 16*q (shift/mask), and one byte-permute
//       per register gathers four consecutive k of one column, which is the
//       operand register of the int8 tensor-core MMA (int8 weights need the
//       permute only);
//   mma.sync m16n8k32 s8 x s8 -> s32: weights are the 16-row operand (16 output
//       columns), activations the 8-column operand.
//
// Activations are fp32 in the API.  Each row of a CTA's K-chunk is scaled by a
// power of two so that max|a| lands in [2^19, 2^20), rounded to an integer and
// written as three signed 7-bit digits (a = d1*2^14 + d2*2^7 + d3), one MMA
// column per digit.  Integer products and sums are exact; the only error is
// the rounding of a to 20 bits relative to the chunk maximum (2^-21), so any
// fp32 input meets the 1e-3 / 1e-4 tolerance against the reference's fp32 loop
// (src/kernels/gemm_quant.cpp:54-82).  int32 partial sums are converted to
// fp32 at every quantisation group (at most every 128 k), multiplied by the
// group scale and accumulated in fp32.
//
// K is split over blockIdx.y.  With 2 or 4 splits the CTAs of a column tile
// form a thread-block cluster and sum their partial [M, 256] tiles in split
// order through distributed shared memory; with other split counts each split
// writes its partial to the context's scratch arena and the last one to arrive
// (a self-resetting counter) sums them in the same order.  Either way the
// result is deterministic and C is written once, with alpha/beta applied.
#include <cooperative_groups.h>

#include <cstdlib>

#include "common.cuh"
#include "dispatch.h"
#include "ptx.cuh"

namespace cg = cooperative_groups;

namespace lhb {

constexpr int GV_BOX_COLS = 128;    // TMA box inner extent (bytes = columns), one 128-byte swizzle row
constexpr int GV_BOXES = 2;         // boxes side by side per stage
constexpr int GV_COLS = GV_BOX_COLS * GV_BOXES;   // columns per CTA
constexpr int GV_ROWS = 64;         // byte-rows per stage
constexpr int GV_BOX_BYTES = GV_BOX_COLS * GV_ROWS;
constexpr int GV_STAGE_BYTES = GV_BOX_BYTES * GV_BOXES;
constexpr int GV_MAX_STAGE = 8;     // ring depth is chosen per launch (2..8) from the shared-memory budget
constexpr int GV_CONSUMER_WARPS = 8;
constexpr int GV_THREADS = (GV_CONSUMER_WARPS + 1) * 32;   // + one producer warp
constexpr int GV_MAX_SPLIT = 32;
constexpr int GV_MAX_M = 16;

using ptx::smem_u32;

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

__device__ __forceinline__ void mma_s8_16832(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// exact int32 -> fp32 for |v| < 2^22 without the conversion pipe
__device__ __forceinline__ float small_int_to_float(int v) {
    return __int_as_float(v + 0x4B400000) - 12582912.0f;
}

struct GemvParams {
    const float* A;        // [M, K]
    const float* scales;   // W4: [K/G, N]   W8: [N]
    float* C;              // [M, N]
    int M, N, K, G;        // G unused for W8
    float alpha, beta;
    int stages_total;      // ceil(rows / 64)
    int stages_per_cta;
    int splits;            // gridDim.y
    int groups_per_cta;    // W4: rows of the shared scale panel (0 for W8)
    float* partial;        // scratch [splits, M, N] (unused when splits == 1)
    int* counters;         // one per column tile, zero between calls
    int* status;
    int nstage;            // ring depth
    int cluster;           // 1: the splits of a column tile form a thread-block cluster (reduce through DSMEM)
    int debug;             // timing experiments only (LHB_GEMV_DEBUG): 1 skip split reduction, 2 skip digits, 4 skip MMAs
};

// WBITS: 4 or 8.  JB: number of 8-column activation blocks; 3 digit columns per
// row of A, so M <= (8 * JB) / 3.
template <int WBITS, int JB>
__global__ void __launch_bounds__(GV_THREADS, (JB >= 6) ? 1 : (JB >= 2 ? 2 : 3))
gemv_mma_kernel(const __grid_constant__ TensorMap tmB, const GemvParams p) {
    constexpr int K_PER_ROW = (WBITS == 4) ? 2 : 1;
    constexpr int K_PER_STAGE = GV_ROWS * K_PER_ROW;
    constexpr int KB_PER_STAGE = K_PER_STAGE / 32;        // k32 blocks per stage: 4 (W4), 2 (W8)
    constexpr int NJ = 8 * JB;                            // digit columns

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int NST = p.nstage;
    uint8_t* tiles = smem;                                             // NST * 16 KiB
    float* part = reinterpret_cast<float*>(smem + NST * GV_STAGE_BYTES);         // [NJ][256]
    float* inv_s = part + NJ * GV_COLS;                                // [16]
    unsigned* rowmax = reinterpret_cast<unsigned*>(inv_s + 16);        // [16] max|a| bits per row
    uint64_t* bars = reinterpret_cast<uint64_t*>(rowmax + 16);         // full[], empty[]
    int* flags = reinterpret_cast<int*>(bars + 2 * GV_MAX_STAGE);      // [0] abort, [1] is-last
    float* sscale = reinterpret_cast<float*>(flags + 4);               // W4: [groups_per_cta][256] group scales
    uint8_t* dfrag = reinterpret_cast<uint8_t*>(sscale + p.groups_per_cta * GV_COLS);   // [kb32][NJ][32]
    volatile int* abort_flag = flags;

    const int ks = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int col0 = blockIdx.x * GV_COLS;

    const int stage_begin = min(ks * p.stages_per_cta, p.stages_total);
    const int stage_end = min(stage_begin + p.stages_per_cta, p.stages_total);
    const int n_stages = stage_end - stage_begin;
    const int k_begin = stage_begin * K_PER_STAGE;
    const int k_count = n_stages * K_PER_STAGE;            // multiple of 32; may run past K

    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + GV_MAX_STAGE);
    // The producer thread sets the barriers up and puts the first ring-full of stages
    // in flight before anything else happens in the CTA.
    if (warp == GV_CONSUMER_WARPS && lane == 0) {
        for (int s = 0; s < GV_MAX_STAGE; ++s) {
            ptx::mbar_init(full0 + 8 * s, 1);
            ptx::mbar_init(empty0 + 8 * s, GV_CONSUMER_WARPS);
        }
        flags[0] = 0;
        flags[1] = 0;
        ptx::fence_mbar_init();
        const int first = min(n_stages, NST);
        for (int s = 0; s < first; ++s) {
            ptx::mbar_expect_tx(full0 + 8 * s, GV_STAGE_BYTES);
#pragma unroll
            for (int b = 0; b < GV_BOXES; ++b)
                ptx::tma_load_2d(smem_u32(tiles + s * GV_STAGE_BYTES + b * GV_BOX_BYTES), &tmB,
                                 col0 + b * GV_BOX_COLS, (stage_begin + s) * GV_ROWS, full0 + 8 * s);
        }
    }
    if (threadIdx.x < 16) rowmax[threadIdx.x] = 0u;
    // Programmatic dependent launch: the weight loads above depend on nothing an
    // earlier kernel in the stream writes, so they are already in flight while
    // that kernel drains; everything below (activations, C, scratch, counters)
    // waits for it to finish.  The next kernel may be scheduled from here on.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __syncthreads();

    // ---- prologue, overlapped with the loads in flight ---------------------------
    // W4: this CTA's panel of group scales, [groups][128 columns], coalesced
    const int g_first = (WBITS == 4) ? k_begin / p.G : 0;
    if (WBITS == 4) {
        for (int i = threadIdx.x; i < p.groups_per_cta * (GV_COLS / 4); i += GV_THREADS) {
            const int gl = i / (GV_COLS / 4), c = (i % (GV_COLS / 4)) * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if ((g_first + gl) * p.G < p.K && col0 + c < p.N)      // N % 16 == 0: whole float4 in range
                v = *reinterpret_cast<const float4*>(p.scales + static_cast<int64_t>(g_first + gl) * p.N + col0 + c);
            *reinterpret_cast<float4*>(sscale + gl * GV_COLS + c) = v;
        }
    }
    // Activations: row maxima of this CTA's K-chunk, then three 7-bit digits per
    // element in MMA-operand order.  Digit columns of rows m >= M are left as
    // they are: an MMA column only feeds its own output column, never read.
    const int q4 = k_count >> 2;                           // float4 per row
    const int n4 = p.M * q4;
    const int n4_pad = (n4 + 31) & ~31;                    // whole warps take part in the shuffles
    const float inv_q4 = 1.0f / static_cast<float>(q4 > 0 ? q4 : 1);
    for (int i = threadIdx.x; i < ((p.debug & 2) ? 0 : n4_pad); i += GV_THREADS) {
        const bool valid = i < n4;
        // row index without an integer division: (i + 0.5) / q4 is never within
        // 0.5 / q4 of an integer, far more than the float error at these sizes
        const int m = valid ? min(p.M - 1, __float2int_rz((static_cast<float>(i) + 0.5f) * inv_q4)) : -1;
        const int k = (i - m * q4) * 4;
        float mx = 0.0f;
        if (valid && k_begin + k < p.K) {
            const float4 v = *reinterpret_cast<const float4*>(p.A + static_cast<int64_t>(m) * p.K + k_begin + k);
            mx = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
        }
        const int m0 = __shfl_sync(0xffffffffu, m, 0);
        if (__all_sync(0xffffffffu, m == m0)) {            // the usual case: one row per warp step
            mx = warp_max(mx);
            if (lane == 0 && m0 >= 0 && mx > 0.0f) atomicMax(rowmax + m0, __float_as_uint(mx));
        } else if (valid && mx > 0.0f) {
            atomicMax(rowmax + m, __float_as_uint(mx));
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < ((p.debug & 2) ? 0 : n4); i += GV_THREADS) {
        const int m = min(p.M - 1, __float2int_rz((static_cast<float>(i) + 0.5f) * inv_q4));
        const int k = (i - m * q4) * 4;
        // power-of-two factor taking max|a| into [2^19, 2^20); exponent clamped
        const unsigned mb = rowmax[m];
        int se = mb ? 273 - static_cast<int>((mb >> 23) & 0xff) : 127;     // 127 + 19 - (e - 127)
        se = max(1, min(253, se));
        const float sc = __uint_as_float(static_cast<uint32_t>(se) << 23);
        if (k == 0) inv_s[m] = __uint_as_float(static_cast<uint32_t>(254 - se) << 23);
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (k_begin + k < p.K)
            v = *reinterpret_cast<const float4*>(p.A + static_cast<int64_t>(m) * p.K + k_begin + k);
        const float x[4] = {v.x * sc, v.y * sc, v.z * sc, v.w * sc};
        uint32_t d1 = 0, d2 = 0, d3 = 0;                  // 4 digits each, one byte per element
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int iv = __float2int_rn(fminf(fmaxf(x[j], -1048576.0f), 1048576.0f));
            const int lo = ((iv + 64) & 127) - 64;
            iv = (iv - lo) >> 7;
            const int mid = ((iv + 64) & 127) - 64;
            const int hi = (iv - mid) >> 7;
            d1 |= static_cast<uint32_t>(hi & 0xff) << (8 * j);
            d2 |= static_cast<uint32_t>(mid & 0xff) << (8 * j);
            d3 |= static_cast<uint32_t>(lo & 0xff) << (8 * j);
        }
        const int kb = k >> 5, kin = k & 31, half = kin >> 4, r = kin & 15;
        uint8_t* base = dfrag + (kb * NJ + 3 * m) * 32 + half * 4;
        if (WBITS == 4) {
            // thread slot t = r / 4 holds k0 + 4t .. 4t+3 (and +16 in the second word)
            uint8_t* d = base + (r >> 2) * 8;
            *reinterpret_cast<uint32_t*>(d) = d1;
            *reinterpret_cast<uint32_t*>(d + 32) = d2;
            *reinterpret_cast<uint32_t*>(d + 64) = d3;
        } else {
            // slot t holds k0 + {2t, 2t+1, 8+2t, 9+2t}: elements (k, k+1) -> slot t0,
            // (k+2, k+3) -> slot t0 + 1, bytes 0-1 (r < 8) or 2-3 (r >= 8)
            uint8_t* d = base + ((r & 7) >> 1) * 8 + ((r >> 3) << 1);
            *reinterpret_cast<uint16_t*>(d) = static_cast<uint16_t>(d1);
            *reinterpret_cast<uint16_t*>(d + 8) = static_cast<uint16_t>(d1 >> 16);
            *reinterpret_cast<uint16_t*>(d + 32) = static_cast<uint16_t>(d2);
            *reinterpret_cast<uint16_t*>(d + 40) = static_cast<uint16_t>(d2 >> 16);
            *reinterpret_cast<uint16_t*>(d + 64) = static_cast<uint16_t>(d3);
            *reinterpret_cast<uint16_t*>(d + 72) = static_cast<uint16_t>(d3 >> 16);
        }
    }
    __syncthreads();

    // ---- main loop ------------------------------------------------------------------
    if (warp < GV_CONSUMER_WARPS) {
        // A warp owns two 16-column fragments f = 0, 1: columns 32*warp + 16*f .. +15 of
        // the CTA, i.e. 16-byte chunks 2*(warp%4) + f of box warp/4.
        const int g = lane >> 2, t = lane & 3;
        const int box = warp >> 2, chunk0 = (warp & 3) * 2;
        const int wcol = warp * 32 + 2 * g;                 // + 16*f: this thread's column pair in the CTA
        float out[2][JB][4];
        int acc[2][JB][4];
#pragma unroll
        for (int f = 0; f < 2; ++f)
#pragma unroll
            for (int jb = 0; jb < JB; ++jb)
#pragma unroll
                for (int i = 0; i < 4; ++i) { out[f][jb][i] = 0.0f; acc[f][jb][i] = 0; }
        // int32 sums are folded into fp32 every `flush_every` k32-blocks: at the end
        // of each quantisation group, and at least every 128 k (keeps |acc| < 2^22)
        const int flush_every = (WBITS == 4) ? min(p.G, 128) / 32 : 4;
        const int group_blocks = (WBITS == 4) ? p.G / 32 : 0x7fffffff;     // k32-blocks per group
        int since_flush = 0;
        int blk_in_group = (WBITS == 4) ? (k_begin / 32) % group_blocks : 0;
        const float* sthread = sscale + wcol;               // + gl * GV_COLS + 16 * f
        const int lrow = lane & 7, lmat = lane >> 3;
        const uint8_t* dthread = dfrag + g * 32 + t * 8;   // + (kb * NJ + jb * 8) * 32

        auto flush = [&]() {
#pragma unroll
            for (int f = 0; f < 2; ++f) {
                float s0 = 1.0f, s1 = 1.0f;
                if (WBITS == 4) {
                    const float2 sv = *reinterpret_cast<const float2*>(sthread + 16 * f);
                    s0 = sv.x; s1 = sv.y;
                }
#pragma unroll
                for (int jb = 0; jb < JB; ++jb) {
                    out[f][jb][0] = fmaf(s0, small_int_to_float(acc[f][jb][0]), out[f][jb][0]);
                    out[f][jb][1] = fmaf(s0, small_int_to_float(acc[f][jb][1]), out[f][jb][1]);
                    out[f][jb][2] = fmaf(s1, small_int_to_float(acc[f][jb][2]), out[f][jb][2]);
                    out[f][jb][3] = fmaf(s1, small_int_to_float(acc[f][jb][3]), out[f][jb][3]);
                    acc[f][jb][0] = acc[f][jb][1] = acc[f][jb][2] = acc[f][jb][3] = 0;
                }
            }
        };
        // one k32-block: the activation fragment is loaded once and feeds both column fragments
        auto mma_block = [&](const uint32_t (&a)[2][4]) {
#pragma unroll
            for (int jb = 0; jb < JB; ++jb) {
                const uint2 b = *reinterpret_cast<const uint2*>(dthread + jb * 8 * 32);
                mma_s8_16832(acc[0][jb], a[0][0], a[0][1], a[0][2], a[0][3], b.x, b.y);
                mma_s8_16832(acc[1][jb], a[1][0], a[1][1], a[1][2], a[1][3], b.x, b.y);
            }
            dthread += NJ * 32;
            ++since_flush;
            ++blk_in_group;
            if (since_flush == flush_every || blk_in_group == group_blocks) { since_flush = 0; flush(); }
            if (blk_in_group == group_blocks) { blk_in_group = 0; sthread += GV_COLS; }
        };

        int slot = 0;
        uint32_t phase = 0;
        for (int ls = 0; ls < n_stages; ++ls) {
            ptx::mbar_wait(full0 + 8 * slot, phase, abort_flag, p.status);
            const uint32_t tile = smem_u32(tiles + slot * GV_STAGE_BYTES + box * GV_BOX_BYTES);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                // register x[f][j]: bytes {row 2t: col 2g, col 2g+1; row 2t+1: col 2g, col 2g+1}
                // of byte-rows 8j .. 8j+7 of this 32-row block, fragment f
                uint32_t x[2][4];
                const int row = half * 32 + lmat * 8 + lrow;
                ldmatrix_x4_trans(tile + row * 128 + (((chunk0) ^ (row & 7)) << 4), x[0]);
                ldmatrix_x4_trans(tile + row * 128 + (((chunk0 + 1) ^ (row & 7)) << 4), x[1]);
                if (half == 1) {           // stage fully read by this warp
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(empty0 + 8 * slot);
                }
                if (p.debug & 4) continue;
                if (WBITS == 4) {
                    uint32_t a[2][2][4];   // [k32-block][fragment][operand register]
#pragma unroll
                    for (int f = 0; f < 2; ++f)
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const uint32_t lo = (x[f][j] << 4) & 0xf0f0f0f0u;     // even k, int8 = 16*q
                            const uint32_t hi = x[f][j] & 0xf0f0f0f0u;            // odd k
                            // 4 consecutive k of column 2g (regs 0, 2) / 2g+1 (regs 1, 3)
                            a[j >> 1][f][(j & 1) * 2] = __byte_perm(lo, hi, 0x6240);
                            a[j >> 1][f][(j & 1) * 2 + 1] = __byte_perm(lo, hi, 0x7351);
                        }
                    mma_block(a[0]);
                    mma_block(a[1]);
                } else {
                    // k-slots 4t..4t+3 <- rows {2t, 2t+1} of matrices 0 and 1; 16+4t.. <- matrices 2 and 3
                    uint32_t a[2][4];
#pragma unroll
                    for (int f = 0; f < 2; ++f) {
                        a[f][0] = __byte_perm(x[f][0], x[f][1], 0x6420);
                        a[f][1] = __byte_perm(x[f][0], x[f][1], 0x7531);
                        a[f][2] = __byte_perm(x[f][2], x[f][3], 0x6420);
                        a[f][3] = __byte_perm(x[f][2], x[f][3], 0x7531);
                    }
                    mma_block(a);
                }
            }
            if (++slot == NST) { slot = 0; phase ^= 1; }
        }
        if (since_flush != 0) flush();
        // per-column partial sums: column j of the operand = digit (j % 3) of row j / 3
#pragma unroll
        for (int f = 0; f < 2; ++f) {
            float c0 = 1.0f, c1 = 1.0f;
            if (WBITS == 8) {
                const int n_a = col0 + wcol + 16 * f;
                c0 = (n_a < p.N) ? p.scales[n_a] : 0.0f;
                c1 = (n_a + 1 < p.N) ? p.scales[n_a + 1] : 0.0f;
            }
#pragma unroll
            for (int jb = 0; jb < JB; ++jb) {
                float* d = part + (jb * 8 + 2 * t) * GV_COLS + wcol + 16 * f;
                *reinterpret_cast<float2*>(d) = make_float2(c0 * out[f][jb][0], c1 * out[f][jb][2]);
                *reinterpret_cast<float2*>(d + GV_COLS) = make_float2(c0 * out[f][jb][1], c1 * out[f][jb][3]);
            }
        }
    } else if (lane == 0) {
        // producer: refill ring slots as the consumers release them
        int issued = min(n_stages, NST);
        int slot = 0;
        uint32_t phase = 0;                                // parity of the consumers' release being waited for
        for (int ls = NST; ls < n_stages; ++ls) {
            if (!ptx::mbar_wait(empty0 + 8 * slot, phase, abort_flag, p.status)) break;
            ptx::mbar_expect_tx(full0 + 8 * slot, GV_STAGE_BYTES);
#pragma unroll
            for (int b = 0; b < GV_BOXES; ++b)
                ptx::tma_load_2d(smem_u32(tiles + slot * GV_STAGE_BYTES + b * GV_BOX_BYTES), &tmB,
                                 col0 + b * GV_BOX_COLS, (stage_begin + ls) * GV_ROWS, full0 + 8 * slot);
            issued = ls + 1;
            if (++slot == NST) { slot = 0; phase ^= 1; }
        }
        if (*abort_flag) {
            // a wait ran out: let the copies still in flight land before the CTA exits
            for (int ls = max(0, issued - NST); ls < issued; ++ls) {
                const uint64_t t0 = ptx::global_timer_ns();
                while (!ptx::mbar_try_wait(full0 + 8 * (ls % NST), (ls / NST) & 1))
                    if (ptx::global_timer_ns() - t0 > 200000000ull) break;
            }
        }
    }
    __syncthreads();

    // ---- combine the three digit columns of every row; write C or the split's partial ----
    const int ncol = min(GV_COLS, p.N - col0);            // multiple of 16
    const float digit_unit = (WBITS == 4) ? 0.0625f : 1.0f;    // int4 nibbles were carried as 16*q
    for (int i = threadIdx.x; i < p.M * (GV_COLS / 4); i += GV_THREADS) {
        const int m = i >> 6, c = (i & 63) * 4;
        if (c >= ncol) continue;
        const float4 h = *reinterpret_cast<const float4*>(part + (3 * m) * GV_COLS + c);
        const float4 md = *reinterpret_cast<const float4*>(part + (3 * m + 1) * GV_COLS + c);
        const float4 l = *reinterpret_cast<const float4*>(part + (3 * m + 2) * GV_COLS + c);
        const float is = inv_s[m] * digit_unit;
        float4 v;
        v.x = is * fmaf(16384.0f, h.x, fmaf(128.0f, md.x, l.x));
        v.y = is * fmaf(16384.0f, h.y, fmaf(128.0f, md.y, l.y));
        v.z = is * fmaf(16384.0f, h.z, fmaf(128.0f, md.z, l.z));
        v.w = is * fmaf(16384.0f, h.w, fmaf(128.0f, md.w, l.w));
        if (p.splits == 1) {
            float4* cp = reinterpret_cast<float4*>(p.C + static_cast<int64_t>(m) * p.N + col0 + c);
            if (p.beta == 0.0f) {
                v.x *= p.alpha; v.y *= p.alpha; v.z *= p.alpha; v.w *= p.alpha;
            } else {
                const float4 o = *cp;
                v.x = fmaf(p.beta, o.x, p.alpha * v.x); v.y = fmaf(p.beta, o.y, p.alpha * v.y);
                v.z = fmaf(p.beta, o.z, p.alpha * v.z); v.w = fmaf(p.beta, o.w, p.alpha * v.w);
            }
            *cp = v;
        } else if (p.cluster) {
            *reinterpret_cast<float4*>(reinterpret_cast<float*>(tiles) + m * GV_COLS + c) = v;   // ring is dead by now
        } else {
            *reinterpret_cast<float4*>(p.partial + (static_cast<int64_t>(ks) * p.M + m) * p.N + col0 + c) = v;
        }
    }
    if (p.splits == 1 || (p.debug & 1)) return;

    if (p.cluster) {
        // Split-K reduction inside the cluster: every CTA finishes a slice of the
        // 256 columns, reading the partial tiles of all splits in split order
        // through distributed shared memory.  No global round trip.
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        const int S = p.splits, rank = static_cast<int>(cluster.block_rank());
        const int q4s = (GV_COLS / 4) / S;                       // float4 columns per CTA (S divides 64)
        const float* comb = reinterpret_cast<const float*>(tiles);
        for (int i = threadIdx.x; i < p.M * q4s; i += GV_THREADS) {
            const int m = i / q4s, c = (rank * q4s + i % q4s) * 4;
            if (c >= ncol) continue;
            float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int r = 0; r < S; ++r) {
                const float4 v = *reinterpret_cast<const float4*>(cluster.map_shared_rank(comb, r) + m * GV_COLS + c);
                sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
            }
            float4* cp = reinterpret_cast<float4*>(p.C + static_cast<int64_t>(m) * p.N + col0 + c);
            if (p.beta == 0.0f) {
                sum.x *= p.alpha; sum.y *= p.alpha; sum.z *= p.alpha; sum.w *= p.alpha;
            } else {
                const float4 o = *cp;
                sum.x = fmaf(p.beta, o.x, p.alpha * sum.x); sum.y = fmaf(p.beta, o.y, p.alpha * sum.y);
                sum.z = fmaf(p.beta, o.z, p.alpha * sum.z); sum.w = fmaf(p.beta, o.w, p.alpha * sum.w);
            }
            *cp = sum;
        }
        cluster.sync();     // keep every CTA's shared memory alive until all peers have read it
        return;
    }

    // Split-K epilogue: the last split to arrive for this column tile sums the
    // partials in split order and writes C.
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int old = atomicAdd(p.counters + blockIdx.x, 1);
        flags[1] = (old == p.splits - 1);
        if (old == p.splits - 1) p.counters[blockIdx.x] = 0;   // ready for the next call
    }
    __syncthreads();
    if (!flags[1]) return;
    __threadfence();
    for (int i = threadIdx.x; i < p.M * (GV_COLS / 4); i += GV_THREADS) {
        const int m = i >> 6, c = (i & 63) * 4;
        if (c >= ncol) continue;
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int r = 0; r < p.splits; ++r) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(
                p.partial + (static_cast<int64_t>(r) * p.M + m) * p.N + col0 + c));
            sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
        }
        float4* cp = reinterpret_cast<float4*>(p.C + static_cast<int64_t>(m) * p.N + col0 + c);
        if (p.beta == 0.0f) {
            sum.x *= p.alpha; sum.y *= p.alpha; sum.z *= p.alpha; sum.w *= p.alpha;
        } else {
            const float4 o = *cp;
            sum.x = fmaf(p.beta, o.x, p.alpha * sum.x); sum.y = fmaf(p.beta, o.y, p.alpha * sum.y);
            sum.z = fmaf(p.beta, o.z, p.alpha * sum.z); sum.w = fmaf(p.beta, o.w, p.alpha * sum.w);
        }
        *cp = sum;
    }
}

// ---- host side --------------------------------------------------------------------

static int gemv_groups_per_cta(int wbits, int k_per_cta, int G) {
    return wbits == 4 ? k_per_cta / G + 2 : 0;             // + 2: chunks need not start on a group boundary
}

// shared memory of a CTA without its ring
static size_t gemv_smem_bytes(int wbits, int jb, int k_per_cta, int G) {
    const size_t nj = 8 * jb;
    return 1024 + nj * GV_COLS * 4 + 16 * 4 + 16 * 4 + 2 * GV_MAX_STAGE * 8 + 16 +
           static_cast<size_t>(gemv_groups_per_cta(wbits, k_per_cta, G)) * GV_COLS * 4 +
           static_cast<size_t>(k_per_cta) * nj;
}

struct GemvPlan { int splits; int stages_total; int stages_per_cta; int nstage; size_t smem; bool ok; };

// Pick the K split.  A CTA costs its stage count plus a fixed overhead (launch,
// activation prologue, partial write-out, about three stages' worth); the grid
// should fit in one wave of the CTAs an SM can hold (3 for M <= 2).  The shared-memory budget (the
// activation digits grow with the chunk length) bounds the chunk from above.
static GemvPlan plan_gemv(int wbits, int jb, int N, int K, int G, int sm_count) {
    GemvPlan best{};
    const int k_per_stage = GV_ROWS * (wbits == 4 ? 2 : 1);
    const int stages_total = ceil_div(K, k_per_stage);
    const int col_tiles = ceil_div(N, GV_COLS);
    double best_cost = 1e30;
    int forced = 0;
    if (const char* e = getenv("LHB_GEMV_SPLITS")) forced = atoi(e);
    for (int S = 1; S <= std::min(stages_total, GV_MAX_SPLIT); ++S) {
        if (forced > 0 && S != std::min(forced, std::min(stages_total, GV_MAX_SPLIT))) continue;
        const int spc = ceil_div(stages_total, S);
        const int splits = ceil_div(stages_total, spc);
        const size_t fixed = gemv_smem_bytes(wbits, jb, spc * k_per_stage, G);
        if (fixed + 2 * GV_STAGE_BYTES > 200 * 1024) continue;
        const int reg_limit = jb >= 6 ? 1 : (jb >= 2 ? 2 : 3);       // CTAs per SM the register file allows
        // CTAs an SM must hold for the grid to be one wave, then the deepest ring that still fits
        int per_sm = std::min(reg_limit, std::max(1, ceil_div(col_tiles * splits, sm_count)));
        while (per_sm > 1 && fixed + 2 * GV_STAGE_BYTES + 1024 > (224 * 1024) / static_cast<size_t>(per_sm)) --per_sm;
        const size_t budget = std::min<size_t>(200 * 1024, (224 * 1024) / per_sm - 1024);
        int nstage = static_cast<int>((budget - fixed) / GV_STAGE_BYTES);
        nstage = std::max(2, std::min(nstage, std::min(spc, GV_MAX_STAGE)));
        const size_t smem = fixed + static_cast<size_t>(nstage) * GV_STAGE_BYTES;
        const int waves = ceil_div(col_tiles * splits, sm_count * per_sm);
        // a shallow ring cannot keep the memory system busy: charge the stages that do not fit
        // the reduction over 2 or 4 splits stays inside a cluster (cheap); other counts go through scratch
        const double red = (splits == 2 || splits == 4) ? 0.6 : 1.2;
        const double cost = waves * (spc + 3.0 + 0.5 * std::max(0, spc - nstage)) + red * splits;
        if (cost < best_cost) {
            best_cost = cost;
            best.splits = splits; best.stages_total = stages_total; best.stages_per_cta = spc;
            best.nstage = nstage; best.smem = smem; best.ok = true;
        }
    }
    return best;
}

static int jb_for(int M) { return M <= 2 ? 1 : (M <= 5 ? 2 : (M <= 8 ? 3 : 6)); }

bool w4a16_fast_ok(int M, int N, int K, int G) {
    if (M < 1 || (N % 16) != 0 || (K % 32) != 0 || (G % 32) != 0 || (K % G) != 0) return false;
    if (G > 128 && (G % 128) != 0) return false;  // int32 sums are folded every 128 k at the latest
    if (M > 64) return false;                     // larger M: generic path (dense GEMM territory)
    return plan_gemv(4, jb_for(std::min(M, GV_MAX_M)), N, K, G, 148).ok;
}

bool w8a16_fast_ok(int M, int N, int K) {
    if (M < 1 || (N % 16) != 0 || (K % 32) != 0) return false;
    if (M > 64) return false;
    return plan_gemv(8, jb_for(std::min(M, GV_MAX_M)), N, K, 1, 148).ok;
}

template <int WBITS, int JB>
static int launch_gemv_t(lhb_ctx* ctx, const TensorMap& tm, GemvParams p, const GemvPlan& pl,
                         cudaStream_t st) {
    auto kern = gemv_mma_kernel<WBITS, JB>;
    static bool attr_set[64] = {};                // per instantiation and device
    if (!attr_set[ctx->device & 63]) {
        LHB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_set[ctx->device & 63] = true;
    }
    p.stages_total = pl.stages_total;
    p.stages_per_cta = pl.stages_per_cta;
    p.splits = pl.splits;
    p.nstage = pl.nstage;
    p.groups_per_cta = gemv_groups_per_cta(WBITS, pl.stages_per_cta * GV_ROWS * (WBITS == 4 ? 2 : 1), p.G);
    p.partial = reinterpret_cast<float*>(ctx->scratch);
    p.counters = ctx->counters;
    p.status = ctx->status_word;
    static const int dbg = getenv("LHB_GEMV_DEBUG") ? atoi(getenv("LHB_GEMV_DEBUG")) : 0;
    p.debug = dbg;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ceil_div(p.N, GV_COLS), pl.splits, 1);
    cfg.blockDim = dim3(GV_THREADS, 1, 1);
    cfg.dynamicSmemBytes = pl.smem;
    cfg.stream = st;
    static const bool pdl = !(getenv("LHB_PDL") && atoi(getenv("LHB_PDL")) == 0);
    static const bool use_cluster = !(getenv("LHB_GEMV_CLUSTER") && atoi(getenv("LHB_GEMV_CLUSTER")) == 0);
    p.cluster = (use_cluster && (pl.splits == 2 || pl.splits == 4)) ? 1 : 0;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    if (p.cluster) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = 1;
        attr[na].val.clusterDim.y = pl.splits;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    LHB_CUDA(cudaLaunchKernelEx(&cfg, kern, tm, p));
    return LHB_OK;
}

template <int WBITS>
static int launch_gemv(lhb_ctx* ctx, const float* A, const void* B, const float* scales, float* C,
                       int M, int N, int K, int G, float alpha, float beta, cudaStream_t st) {
    const uint64_t rows = (WBITS == 4) ? K / 2 : K;
    TensorMap tm;
    if (int e = get_tensor_map_2d_u8(ctx, B, rows, N, N, GV_ROWS, GV_BOX_COLS, true, &tm)) return e;
    // rows of A are independent: M > 16 is served in slabs of 16 rows
    for (int m0 = 0; m0 < M; m0 += GV_MAX_M) {
        const int m = std::min(GV_MAX_M, M - m0);
        const int jb = jb_for(m);
        GemvPlan pl = plan_gemv(WBITS, jb, N, K, WBITS == 4 ? G : 1, ctx->sm_count);
        if (!pl.ok) return LHB_ERR_UNSUPPORTED;
        if (ceil_div(N, GV_COLS) > static_cast<int>(ctx->counters_len)) return LHB_ERR_UNSUPPORTED;
        if (pl.splits > 1 && static_cast<size_t>(pl.splits) * m * N * sizeof(float) > ctx->scratch_bytes)
            return LHB_ERR_SCRATCH;
        GemvParams p{};
        p.A = A + static_cast<int64_t>(m0) * K;
        p.scales = scales;
        p.C = C + static_cast<int64_t>(m0) * N;
        p.M = m; p.N = N; p.K = K; p.G = G; p.alpha = alpha; p.beta = beta;
        int e;
        if (jb == 1) e = launch_gemv_t<WBITS, 1>(ctx, tm, p, pl, st);
        else if (jb == 2) e = launch_gemv_t<WBITS, 2>(ctx, tm, p, pl, st);
        else if (jb == 3) e = launch_gemv_t<WBITS, 3>(ctx, tm, p, pl, st);
        else e = launch_gemv_t<WBITS, 6>(ctx, tm, p, pl, st);
        if (e) return e;
    }
    return LHB_OK;
}

int launch_w4a16_fast(lhb_ctx* ctx, const float* A, const uint8_t* Bp, const float* Bs, float* C,
                      int M, int N, int K, int G, float alpha, float beta, cudaStream_t st) {
    return launch_gemv<4>(ctx, A, Bp, Bs, C, M, N, K, G, alpha, beta, st);
}

int launch_w8a16_fast(lhb_ctx* ctx, const float* A, const int8_t* Bq, const float* Bs, float* C,
                      int M, int N, int K, float alpha, float beta, cudaStream_t st) {
    return launch_gemv<8>(ctx, A, Bq, Bs, C, M, N, K, 0, alpha, beta, st);
}

}  // namespace lhb

// Skinny weight-only GEMMs (decode GEMV, M <= 16 per launch) for int4-group
// and int8-per-channel weights in the reference's own layouts:
//   W4: packed uint8 [K/2, N], byte (k/2, n), low nibble = even k
//       (src/kernels/quant.hpp:52-57), fp32 scales [K/G, N];
//   W8: int8 [K, N], fp32 scales [N] (src/kernels/quant.hpp:45-48).
// Both layouts are N-contiguous, i.e. the reduction axis is the slow axis.
//
// The path is HBM-bound: the weight bytes are read exactly once.  To keep the
// instruction count per weight well under what the memory system can feed,
// the dot products run on the tensor cores with the weights dequantised in
// registers:
//
//   TMA (2-D, 128-byte swizzle)  global -> shared, 64 rows x 128 columns per
//       stage, the whole K-chunk of a CTA in flight at once (4-deep ring);
//   ldmatrix.trans on the raw bytes: one 8x8 b16 matrix = 8 byte-rows x 16
//       columns; the transposed fragment hands every thread bytes of ONE
//       column at two consecutive rows, which is exactly the "two adjacent k
//       of one output column" pairing an m16n8k16 A-fragment register needs;
//   nibble/byte -> fp16 with mask+xor against 0x6400 (1024 + x) and one
//       HSUB2/HFMA2, exact for |q| <= 128;
//   mma.sync m16n8k16 f16 x f16 -> f32 with the weights as the 16-row operand
//       (16 output columns) and the activations as the 8-column operand.
//
// Activations are fp32 in the API.  They are split on the fly into two fp16
// terms hi + lo (after an exact power-of-two scaling of each row chunk into
// fp16 range), which occupy two MMA columns per row of A; products and sums
// stay in fp32, so the result differs from the reference's fp32 loop only by
// summation order (~1e-6 relative).
//
// K is split over blockIdx.y so that every SM holds 3-4 CTAs with their whole
// K-chunk in flight.  Each split writes its partial [M, 128] tile to the
// context's scratch arena; the last split to arrive for a column tile (a
// self-resetting counter) sums the partials in fixed order and applies
// alpha/beta, so the result is deterministic and C is written once.
#include <cuda_fp16.h>

#include <cstdlib>

#include "common.cuh"
#include "dispatch.h"
#include "ptx.cuh"

namespace lhb {

constexpr int GV_COLS = 128;        // columns per CTA (TMA box inner extent, bytes)
constexpr int GV_ROWS = 64;         // byte-rows per stage
constexpr int GV_STAGE_BYTES = GV_COLS * GV_ROWS;
constexpr int GV_NSTAGE = 4;
constexpr int GV_CONSUMER_WARPS = 8;
constexpr int GV_THREADS = (GV_CONSUMER_WARPS + 1) * 32;   // + one producer warp
constexpr int GV_MAX_SPLIT = 32;

// ---- PTX wrappers (mbarrier / TMA live in ptx.cuh) --------------------------------

using ptx::smem_u32;

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

// Two int4 nibbles (bits 0-3 of each 16-bit half of `w`, two's complement) ->
// exact fp16 pair: (nib ^ 8) | 0x6400 is the fp16 number 1032 + q.
__device__ __forceinline__ uint32_t nib_lo_to_h2(uint32_t w) {
    const uint32_t t = (w & 0x000f000fu) ^ 0x64086408u;
    return h2_as_u32(__hsub2(u32_as_h2(t), u32_as_h2(0x64086408u)));
}
// Nibbles in bits 4-7 of each half: ((w & 0xf0) ^ 0x80) | 0x6400 = 1152 + 16 q;
// one fused multiply-add (x/16 - 72) gives q exactly.
__device__ __forceinline__ uint32_t nib_hi_to_h2(uint32_t w) {
    const uint32_t t = (w & 0x00f000f0u) ^ 0x64806480u;
    return h2_as_u32(__hfma2(u32_as_h2(t), u32_as_h2(0x2c002c00u) /* 1/16 */,
                             u32_as_h2(0xd480d480u) /* -72 */));
}
// Two int8 values in bytes `sel` of w (already xor 0x80) -> exact fp16 pair:
// byte | 0x6400 is 1024 + (q + 128).
template <uint32_t SEL>
__device__ __forceinline__ uint32_t i8pair_to_h2(uint32_t w_biased) {
    const uint32_t t = __byte_perm(w_biased, 0x64646464u, SEL);
    return h2_as_u32(__hsub2(u32_as_h2(t), u32_as_h2(0x64806480u)));
}

// ---- the kernel ----------------------------------------------------------------

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
};

// WBITS: 4 or 8.  JB: number of 8-column activation blocks (M <= 4*JB).
template <int WBITS, int JB>
__global__ void __launch_bounds__(GV_THREADS, (JB == 4) ? 3 : 4)
gemv_mma_kernel(const __grid_constant__ TensorMap tmB, const GemvParams p) {
    constexpr int K_PER_ROW = (WBITS == 4) ? 2 : 1;
    constexpr int K_PER_STAGE = GV_ROWS * K_PER_ROW;
    constexpr int KB_PER_STAGE = K_PER_STAGE / 16;        // k16 blocks per stage: 8 (W4), 4 (W8)
    constexpr int NJ = 8 * JB;                            // activation columns (2 per row of A)
    constexpr int MROWS = 4 * JB;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* tiles = smem;                                             // GV_NSTAGE * 8 KiB
    float* part = reinterpret_cast<float*>(smem + GV_NSTAGE * GV_STAGE_BYTES);   // [MROWS][128]
    float* inv_s = part + MROWS * GV_COLS;                             // [16]
    unsigned* rowmax = reinterpret_cast<unsigned*>(inv_s + 16);        // [16] max|a| bits per row
    uint64_t* bars = reinterpret_cast<uint64_t*>(rowmax + 16);         // full[4], empty[4]
    int* flags = reinterpret_cast<int*>(bars + 2 * GV_NSTAGE);         // [0] abort, [1] is-last
    float* sscale = reinterpret_cast<float*>(flags + 4);               // W4: [groups_per_cta][128] group scales
    __half* bfrag = reinterpret_cast<__half*>(sscale + p.groups_per_cta * GV_COLS);   // [kb][NJ][4][4]
    volatile int* abort_flag = flags;

    const int ks = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int col0 = blockIdx.x * GV_COLS;

    const int stage_begin = min(ks * p.stages_per_cta, p.stages_total);
    const int stage_end = min(stage_begin + p.stages_per_cta, p.stages_total);
    const int n_stages = stage_end - stage_begin;
    const int k_begin = stage_begin * K_PER_STAGE;
    const int k_count = n_stages * K_PER_STAGE;            // multiple of 16; may run past K

    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + GV_NSTAGE);
    // The producer thread sets the barriers up and puts the first GV_NSTAGE stages
    // in flight before anything else happens in the CTA.
    if (warp == GV_CONSUMER_WARPS && lane == 0) {
        for (int s = 0; s < GV_NSTAGE; ++s) {
            ptx::mbar_init(full0 + 8 * s, 1);
            ptx::mbar_init(empty0 + 8 * s, GV_CONSUMER_WARPS);
        }
        flags[0] = 0;
        flags[1] = 0;
        ptx::fence_mbar_init();
        const int first = min(n_stages, GV_NSTAGE);
        for (int s = 0; s < first; ++s) {
            ptx::mbar_expect_tx(full0 + 8 * s, GV_STAGE_BYTES);
            ptx::tma_load_2d(smem_u32(tiles + s * GV_STAGE_BYTES), &tmB, col0, (stage_begin + s) * GV_ROWS,
                             full0 + 8 * s);
        }
    }
    if (threadIdx.x < 16) rowmax[threadIdx.x] = 0u;
    __syncthreads();

    // Activation prologue (all threads, overlapped with the loads in flight):
    // every live row of this CTA's K-chunk is scaled by a power of two into fp16
    // range, split into hi + lo and stored in B-fragment order.  Columns of rows
    // m >= M are left as they are: an MMA column only feeds its own output
    // column, and those are never read.
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
    const int q4 = k_count >> 2;                           // float4 per row
    const int n4 = p.M * q4;
    for (int i = threadIdx.x; i < n4; i += GV_THREADS) {
        const int m = i / q4, k = (i - m * q4) * 4;
        float mx = 0.0f;
        if (k_begin + k < p.K) {
            const float4 v = *reinterpret_cast<const float4*>(p.A + static_cast<int64_t>(m) * p.K + k_begin + k);
            mx = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
        }
        if (mx > 0.0f) atomicMax(rowmax + m, __float_as_uint(mx));
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n4; i += GV_THREADS) {
        const int m = i / q4, k = (i - m * q4) * 4;
        // power-of-two factor taking max|a| into [2^13, 2^14); exponent clamped
        const unsigned mb = rowmax[m];
        int se = mb ? 267 - static_cast<int>((mb >> 23) & 0xff) : 127;
        se = max(1, min(253, se));
        const float sc = __uint_as_float(static_cast<uint32_t>(se) << 23);
        if (k == 0) inv_s[m] = __uint_as_float(static_cast<uint32_t>(254 - se) << 23);
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (k_begin + k < p.K)
            v = *reinterpret_cast<const float4*>(p.A + static_cast<int64_t>(m) * p.K + k_begin + k);
        const float x[4] = {v.x * sc, v.y * sc, v.z * sc, v.w * sc};
        unsigned short hi[4], lo[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const __half h = __float2half_rn(x[j]);
            hi[j] = __half_as_ushort(h);
            lo[j] = __half_as_ushort(__float2half_rn(x[j] - __half2float(h)));
        }
        const int kb = k >> 4, kin = k & 15;
        if (WBITS == 4) {
            // fragment slot t = kin/4 holds k+{0,2,1,3}: one 8-byte store per column
            __half* d = bfrag + ((kb * NJ + 2 * m) * 4 + (kin >> 2)) * 4;
            *reinterpret_cast<uint2*>(d) = make_uint2(hi[0] | (static_cast<uint32_t>(hi[2]) << 16),
                                                      hi[1] | (static_cast<uint32_t>(hi[3]) << 16));
            *reinterpret_cast<uint2*>(d + 16) = make_uint2(lo[0] | (static_cast<uint32_t>(lo[2]) << 16),
                                                           lo[1] | (static_cast<uint32_t>(lo[3]) << 16));
        } else {
            // slot t holds k0+{2t, 2t+1, 8+2t, 9+2t}: (k, k+1) and (k+2, k+3) go to slots t, t+1
            const int t0 = (kin & 7) >> 1, e = (kin >> 3) << 1;
            __half* d = bfrag + ((kb * NJ + 2 * m) * 4 + t0) * 4 + e;
            *reinterpret_cast<uint32_t*>(d) = hi[0] | (static_cast<uint32_t>(hi[1]) << 16);
            *reinterpret_cast<uint32_t*>(d + 4) = hi[2] | (static_cast<uint32_t>(hi[3]) << 16);
            *reinterpret_cast<uint32_t*>(d + 16) = lo[0] | (static_cast<uint32_t>(lo[1]) << 16);
            *reinterpret_cast<uint32_t*>(d + 20) = lo[2] | (static_cast<uint32_t>(lo[3]) << 16);
        }
    }
    __syncthreads();

    float out[JB][4];
#pragma unroll
    for (int jb = 0; jb < JB; ++jb)
#pragma unroll
        for (int i = 0; i < 4; ++i) out[jb][i] = 0.0f;

    if (warp < GV_CONSUMER_WARPS) {
        const int g = lane >> 2, t = lane & 3;
        const int n_a = col0 + warp * 16 + 2 * g;           // this thread's two output columns
        float acc[JB][4];
#pragma unroll
        for (int jb = 0; jb < JB; ++jb)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[jb][i] = 0.0f;
        float ch0 = 0.0f, ch1 = 0.0f;                      // W8: per-channel scales, fetched ahead of the loop
        if (WBITS == 8) {
            if (n_a < p.N) ch0 = p.scales[n_a];
            if (n_a + 1 < p.N) ch1 = p.scales[n_a + 1];
        }
        const int kb_per_group = (WBITS == 4) ? p.G / 16 : 0x7fffffff;
        int kb_in_group = (WBITS == 4) ? (k_begin / 16) % kb_per_group : 0;
        // ldmatrix row address: matrix (lane / 8), row (lane % 8); 16-byte chunk = warp, swizzled
        const int lrow = lane & 7, lmat = lane >> 3;
        // end of a quantisation group (or of this CTA's chunk): fold the scale
        // of the group that k16-block `kb` belongs to into the running output
        auto flush_group = [&](int kb) {
            const int gl = (k_begin + kb * 16) / p.G - g_first;
            const float2 sv = *reinterpret_cast<const float2*>(sscale + gl * GV_COLS + warp * 16 + 2 * g);
            const float s0 = sv.x, s1 = sv.y;
#pragma unroll
            for (int jb = 0; jb < JB; ++jb) {
                out[jb][0] = fmaf(s0, acc[jb][0], out[jb][0]);
                out[jb][1] = fmaf(s0, acc[jb][1], out[jb][1]);
                out[jb][2] = fmaf(s1, acc[jb][2], out[jb][2]);
                out[jb][3] = fmaf(s1, acc[jb][3], out[jb][3]);
                acc[jb][0] = acc[jb][1] = acc[jb][2] = acc[jb][3] = 0.0f;
            }
        };

        for (int ls = 0; ls < n_stages; ++ls) {
            const int slot = ls % GV_NSTAGE;
            ptx::mbar_wait(full0 + 8 * slot, (ls / GV_NSTAGE) & 1, abort_flag, p.status);
            const uint32_t tile = smem_u32(tiles + slot * GV_STAGE_BYTES);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                uint32_t x[4];
                const int row = half * 32 + lmat * 8 + lrow;
                ldmatrix_x4_trans(tile + row * 128 + ((warp ^ (row & 7)) << 4), x);
                if (half == 1) {           // stage fully read by this warp
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(empty0 + 8 * slot);
                }
                if (WBITS == 4) {
#pragma unroll
                    for (int mat = 0; mat < 4; ++mat) {
                        const int kb = ls * KB_PER_STAGE + half * 4 + mat;
                        const uint32_t a0 = nib_lo_to_h2(x[mat]);
                        const uint32_t a2 = nib_hi_to_h2(x[mat]);
                        const uint32_t a1 = nib_lo_to_h2(x[mat] >> 8);
                        const uint32_t a3 = nib_hi_to_h2(x[mat] >> 8);
#pragma unroll
                        for (int jb = 0; jb < JB; ++jb) {
                            const uint2 b = *reinterpret_cast<const uint2*>(
                                bfrag + ((kb * NJ + jb * 8 + g) * 4 + t) * 4);
                            mma_16816(acc[jb], a0, a1, a2, a3, b.x, b.y);
                        }
                        if (++kb_in_group == kb_per_group) {
                            kb_in_group = 0;
                            flush_group(kb);
                        }
                    }
                } else {
#pragma unroll
                    for (int pr = 0; pr < 2; ++pr) {
                        const int kb = ls * KB_PER_STAGE + half * 2 + pr;
                        const uint32_t w0 = x[2 * pr] ^ 0x80808080u;
                        const uint32_t w1 = x[2 * pr + 1] ^ 0x80808080u;
                        const uint32_t a0 = i8pair_to_h2<0x4240>(w0);
                        const uint32_t a1 = i8pair_to_h2<0x4341>(w0);
                        const uint32_t a2 = i8pair_to_h2<0x4240>(w1);
                        const uint32_t a3 = i8pair_to_h2<0x4341>(w1);
#pragma unroll
                        for (int jb = 0; jb < JB; ++jb) {
                            const uint2 b = *reinterpret_cast<const uint2*>(
                                bfrag + ((kb * NJ + jb * 8 + g) * 4 + t) * 4);
                            mma_16816(acc[jb], a0, a1, a2, a3, b.x, b.y);
                        }
                    }
                }
            }
        }
        if (WBITS == 4 && kb_in_group != 0 && n_stages > 0) flush_group(n_stages * KB_PER_STAGE - 1);
        if (WBITS == 8) {
            const float s0 = ch0, s1 = ch1;
#pragma unroll
            for (int jb = 0; jb < JB; ++jb) {
                out[jb][0] = s0 * acc[jb][0]; out[jb][1] = s0 * acc[jb][1];
                out[jb][2] = s1 * acc[jb][2]; out[jb][3] = s1 * acc[jb][3];
            }
        }
        // hi + lo columns of row m = 4*jb + t, undo the activation scaling; rows of
        // this split go straight to C (one split) or to the scratch partials
#pragma unroll
        for (int jb = 0; jb < JB; ++jb) {
            const int m = 4 * jb + t;
            if (m < p.M && n_a < p.N) {
                const float is = inv_s[m];
                float2 v;
                v.x = is * (out[jb][0] + out[jb][1]);
                v.y = is * (out[jb][2] + out[jb][3]);
                if (p.splits == 1) {
                    float* cp = p.C + static_cast<int64_t>(m) * p.N + n_a;
                    if (p.beta == 0.0f) { v.x *= p.alpha; v.y *= p.alpha; }
                    else { v.x = fmaf(p.beta, cp[0], p.alpha * v.x); v.y = fmaf(p.beta, cp[1], p.alpha * v.y); }
                    *reinterpret_cast<float2*>(cp) = v;       // N % 16 == 0: both columns exist, 8-byte aligned
                } else {
                    *reinterpret_cast<float2*>(p.partial + (static_cast<int64_t>(ks) * p.M + m) * p.N + n_a) = v;
                }
            }
        }
    } else if (lane == 0) {
        // producer: refill ring slots as the consumers release them
        int issued = min(n_stages, GV_NSTAGE);
        for (int ls = GV_NSTAGE; ls < n_stages; ++ls) {
            const int slot = ls % GV_NSTAGE;
            if (!ptx::mbar_wait(empty0 + 8 * slot, ((ls / GV_NSTAGE) - 1) & 1, abort_flag, p.status)) break;
            ptx::mbar_expect_tx(full0 + 8 * slot, GV_STAGE_BYTES);
            ptx::tma_load_2d(smem_u32(tiles + slot * GV_STAGE_BYTES), &tmB, col0,
                             (stage_begin + ls) * GV_ROWS, full0 + 8 * slot);
            issued = ls + 1;
        }
        if (*abort_flag) {
            // a wait ran out: let the copies still in flight land before the CTA exits
            for (int ls = max(0, issued - GV_NSTAGE); ls < issued; ++ls) {
                const uint64_t t0 = ptx::global_timer_ns();
                while (!ptx::mbar_try_wait(full0 + 8 * (ls % GV_NSTAGE), (ls / GV_NSTAGE) & 1))
                    if (ptx::global_timer_ns() - t0 > 200000000ull) break;
            }
        }
    }
    if (p.splits == 1) return;

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
    const int ncol = min(GV_COLS, p.N - col0);
    for (int i = threadIdx.x; i < p.M * (ncol >> 2); i += GV_THREADS) {
        const int m = i / (ncol >> 2), c = (i % (ncol >> 2)) * 4;
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

static size_t gemv_smem_bytes(int wbits, int jb, int k_per_cta, int G) {
    const size_t nj = 8 * jb, mrows = 4 * jb;
    return 1024 + GV_NSTAGE * GV_STAGE_BYTES + mrows * GV_COLS * 4 + 16 * 4 + 16 * 4 + 2 * GV_NSTAGE * 8 + 16 +
           static_cast<size_t>(gemv_groups_per_cta(wbits, k_per_cta, G)) * GV_COLS * 4 +
           static_cast<size_t>(k_per_cta) * nj * 2;
}

struct GemvPlan { int splits; int stages_total; int stages_per_cta; size_t smem; bool ok; };

// Pick the K split.  A CTA costs its stage count plus a fixed overhead (launch,
// activation prologue, partial write-out, about three stages' worth); the grid
// should fit in one wave of ~4 CTAs per SM.  The shared-memory budget (the
// activation fragments grow with the chunk length) bounds the chunk from above.
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
        const size_t smem = gemv_smem_bytes(wbits, jb, spc * k_per_stage, G);
        if (smem > 200 * 1024) continue;
        const int per_sm = std::max(1, std::min(4, static_cast<int>((220 * 1024) / smem)));
        const int waves = ceil_div(col_tiles * splits, sm_count * per_sm);
        const double cost = waves * (spc + 3.0) + 0.05 * splits;
        if (cost < best_cost) {
            best_cost = cost;
            best.splits = splits; best.stages_total = stages_total; best.stages_per_cta = spc;
            best.smem = smem; best.ok = true;
        }
    }
    return best;
}

static int jb_for(int M) { return M <= 4 ? 1 : (M <= 8 ? 2 : 4); }

bool w4a16_fast_ok(int M, int N, int K, int G) {
    if (M < 1 || (N % 16) != 0 || (K % 16) != 0 || (G % 16) != 0 || (K % G) != 0) return false;
    if (M > 64) return false;                     // larger M: generic path (dense GEMM territory)
    return plan_gemv(4, jb_for(M > 16 ? 16 : M), N, K, G, 148).ok;
}

bool w8a16_fast_ok(int M, int N, int K) {
    if (M < 1 || (N % 16) != 0 || (K % 16) != 0) return false;
    if (M > 64) return false;
    return plan_gemv(8, jb_for(M > 16 ? 16 : M), N, K, 1, 148).ok;
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
    p.groups_per_cta = gemv_groups_per_cta(WBITS, pl.stages_per_cta * GV_ROWS * (WBITS == 4 ? 2 : 1), p.G);
    p.partial = reinterpret_cast<float*>(ctx->scratch);
    p.counters = ctx->counters;
    p.status = ctx->status_word;
    const dim3 grid(ceil_div(p.N, GV_COLS), pl.splits, 1);
    kern<<<grid, GV_THREADS, pl.smem, st>>>(tm, p);
    LHB_LAUNCH_CHECK();
    return LHB_OK;
}

template <int WBITS>
static int launch_gemv(lhb_ctx* ctx, const float* A, const void* B, const float* scales, float* C,
                       int M, int N, int K, int G, float alpha, float beta, cudaStream_t st) {
    const uint64_t rows = (WBITS == 4) ? K / 2 : K;
    TensorMap tm;
    if (int e = get_tensor_map_2d_u8(ctx, B, rows, N, N, GV_ROWS, GV_COLS, true, &tm)) return e;
    // rows of A are independent: M > 16 is served in slabs of 16 rows
    for (int m0 = 0; m0 < M; m0 += 16) {
        const int m = std::min(16, M - m0);
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
        else e = launch_gemv_t<WBITS, 4>(ctx, tm, p, pl, st);
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

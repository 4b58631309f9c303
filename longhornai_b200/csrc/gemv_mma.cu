// Skinny weight-only GEMMs (decode GEMV, M <= 16 per launch) for int4-group
// and int8-per-channel weights in the reference's own layouts:
//   W4: packed uint8 [K/2, N], byte (k/2, n), low nibble = even k
//       (src/kernels/quant.hpp:52-57), fp32 scales [K/G, N];
//   W8: int8 [K, N], fp32 scales [N] (src/kernels/quant.hpp:45-48).
// Both layouts are N-contiguous, i.e. the reduction axis is the slow axis.
//
// The path is HBM-bound: the weight bytes are read exactly once, so the kernel
// is built to spend as few issue slots per weight as possible and to give
// every SM the same number of bytes.
//
//   Work units.  The weight matrix is cut into units of 64 byte-rows x 256
//       columns (16 KiB; 128 k of int4 or 64 k of int8).  Units are numbered
//       column tile by column tile, and CTA c of P takes the contiguous range
//       [c*U/P, (c+1)*U/P): every CTA streams the same amount (+-1 unit)
//       whatever N and K are.  With fewer column tiles than CTAs, P is a
//       multiple of the tile count, so a range is a K-slice of one tile; else a
//       range crosses a few tiles and each piece ("segment") is handled in turn.
//   TMA (2-D, 128-byte swizzle) brings a unit into a ring of shared-memory
//       stages; for W4 a second, unswizzled tensor map brings the unit's rows of
//       group scales along on the same barrier.  One producer thread runs ahead
//       of the consumers across segment borders.
//   ldmatrix.trans on the raw bytes: one 8x8 b16 matrix = 8 byte-rows x 16
//       columns; the transposed fragment hands every thread the bytes of two
//       adjacent columns at two consecutive rows.
//   One byte-permute over two such registers gathers four byte-rows of one
//       column.  For int4 that register holds eight weights: masking keeps the
//       odd-k nibbles where they are, shift+mask moves the even-k nibbles up,
//       and a nibble at the top of its byte IS the int8 value 16*q.  These
//       registers are tensor-core operands as they stand: the k order inside a
//       32-block is free as long as the activation operand uses the same order.
//   mma.sync m16n8k32 s8 x s8 -> s32: weights are the 16-row operand (16 output
//       columns), activations the 8-column operand.
//
// Activations are fp32 in the API.  Each row of the K-range a CTA touches is
// scaled by a power of two so that max|a| lands in [2^21, 2^22), rounded to an
// integer and written as three signed 8-bit digits (a = d1*2^16 + d2*2^8 + d3),
// one MMA column per digit.  Integer products and sums are exact; the only error
// is the rounding of a to 22 bits relative to the range maximum (2^-23), so any
// fp32 input meets the 1e-3 / 1e-4 tolerance against the reference's fp32 loop
// (src/kernels/gemm_quant.cpp:54-82).  int32 partial sums are converted to
// fp32 at every quantisation group (at most every 128 k of int4, 256 k of
// int8), multiplied by the group scale and accumulated in fp32.
//
// A segment that covers all of K writes C directly.  Otherwise it writes its
// partial [M, 256] tile to the context's scratch arena, and the last
// contributor to arrive for that column tile (a self-resetting counter) sums
// the partials in contributor order and writes C: deterministic for a given SM
// count, and C is written once, with alpha/beta applied.
#include <cuda_fp16.h>

#include <cstdlib>

#include "common.cuh"
#include "dispatch.h"
#include "ptx.cuh"

namespace lhb {

constexpr int GV_BOX_COLS = 128;    // TMA box inner extent (bytes = columns), one 128-byte swizzle row
constexpr int GV_BOXES = 2;         // boxes side by side per stage
constexpr int GV_COLS = GV_BOX_COLS * GV_BOXES;   // columns per CTA
constexpr int GV_ROWS = 64;         // byte-rows per stage
constexpr int GV_BOX_BYTES = GV_BOX_COLS * GV_ROWS;
constexpr int GV_STAGE_BYTES = GV_BOX_BYTES * GV_BOXES;
constexpr int GV_MAX_STAGE = 8;     // ring depth is chosen per launch (2..8) from the shared-memory budget
constexpr int GV_COL_WARPS = 8;                   // consumer warps across the 256 columns of a tile
// For M > 8 two groups of column warps share a tile: both unpack the same weights, each
// feeds half of the activation digit columns (half the accumulators per warp, twice the
// warps in flight).
constexpr int gv_groups(int jb) { return jb >= 6 ? 2 : 1; }
constexpr int gv_consumer_warps(int jb) { return GV_COL_WARPS * gv_groups(jb); }
constexpr int gv_threads(int jb) { return (gv_consumer_warps(jb) + 1) * 32; }   // + one producer warp
constexpr int GV_MAX_M = 16;
constexpr size_t GV_DIG_BYTES = size_t(4) << 20;   // head of the scratch arena: activation digits of a pass + its row factors
constexpr size_t GV_INV_BYTES = 4096;              // the last 4 KiB of it: one fp32 factor per row, up to 1024 rows a pass
constexpr int GV_PB = 8;           // activation float4 loads a thread keeps in flight in the prologue

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

// the same with C = 0: starts a fresh sum without a separate clearing of the accumulators
__device__ __forceinline__ void mma_s8_16832_first(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                   uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%10,%10,%10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// unsigned weights (asymmetric int4 carried as 16*u in [0, 240]) x signed activation digits
__device__ __forceinline__ void mma_u8s8_16832(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_u8s8_16832_first(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                     uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%10,%10,%10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// barrier among the consumer warps only (the producer warp never joins it)
template <int CONSUMERS>
__device__ __forceinline__ void consumer_sync() {
    asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS) : "memory");
}

// exact int32 -> fp32 for |v| < 2^22 without the conversion pipe
__device__ __forceinline__ float small_int_to_float(int v) {
    return __int_as_float(v + 0x4B400000) - 12582912.0f;
}

// Development aid, compiled only with -DLHB_GEMV_TRACE: thread 0 of every CTA stamps
// %globaltimer at the phase borders of the last 64 launches.
#ifdef LHB_GEMV_TRACE
__device__ unsigned long long g_gv_trace[64][512][8];
#define GV_STAMP(i)                                                                                  \
    do {                                                                                             \
        if (threadIdx.x == 0 && blockIdx.x < 512) g_gv_trace[p.trace_slot][blockIdx.x][i] = ptx::global_timer_ns(); \
    } while (0)
#else
#define GV_STAMP(i) do { } while (0)
#endif

// Three signed 8-bit digits of four consecutive activations (k .. k+3, k % 4 == 0, `kin`
// = k % 32), written into the operand fragment of their k32-block: `base` points at the 32
// bytes of the row's first digit column, the other two follow at +32 and +64.
template <int WBITS>
__device__ __forceinline__ void write_digits(uint8_t* base, int kin, float4 v, float scl) {
    const int half = kin >> 4, r = kin & 15;
    // a = rint(v * scl) = d1*2^16 + d2*2^8 + d3 with d2, d3 in [-128, 127] and |d1| <= 64
    // (|a| <= 2^22): the low byte of an integer, read as signed, is its balanced digit, and
    // what remains is divisible by 256.
    const float x[4] = {v.x * scl, v.y * scl, v.z * scl, v.w * scl};
    uint32_t b1[4], b2[4], b3[4];                     // low byte = digit
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int iv = __float2int_rn(x[j]);
        const int lo = static_cast<int>(static_cast<int8_t>(iv));
        const int iv2 = (iv - lo) >> 8;
        const int mid = static_cast<int>(static_cast<int8_t>(iv2));
        b3[j] = static_cast<uint32_t>(lo);
        b2[j] = static_cast<uint32_t>(mid);
        b1[j] = static_cast<uint32_t>((iv2 - mid) >> 8);
    }
    // d1/d2/d3: 4 digits each, one byte per element
    const uint32_t d1 = __byte_perm(__byte_perm(b1[0], b1[1], 0x0040), __byte_perm(b1[2], b1[3], 0x0040), 0x5410);
    const uint32_t d2 = __byte_perm(__byte_perm(b2[0], b2[1], 0x0040), __byte_perm(b2[2], b2[3], 0x0040), 0x5410);
    const uint32_t d3 = __byte_perm(__byte_perm(b3[0], b3[1], 0x0040), __byte_perm(b3[2], b3[3], 0x0040), 0x5410);
    if (WBITS == 4) {
        // Operand slot order of a k32-block (see the main loop): thread slot t = r / 4,
        // first word = even k {4t, 4t+2, 16+4t, 16+4t+2}, second word = the odd k beside them.
        uint8_t* d = base + (r >> 2) * 8 + half * 2;
        *reinterpret_cast<uint16_t*>(d) = static_cast<uint16_t>(__byte_perm(d1, 0, 0x4420));
        *reinterpret_cast<uint16_t*>(d + 4) = static_cast<uint16_t>(__byte_perm(d1, 0, 0x4431));
        *reinterpret_cast<uint16_t*>(d + 32) = static_cast<uint16_t>(__byte_perm(d2, 0, 0x4420));
        *reinterpret_cast<uint16_t*>(d + 36) = static_cast<uint16_t>(__byte_perm(d2, 0, 0x4431));
        *reinterpret_cast<uint16_t*>(d + 64) = static_cast<uint16_t>(__byte_perm(d3, 0, 0x4420));
        *reinterpret_cast<uint16_t*>(d + 68) = static_cast<uint16_t>(__byte_perm(d3, 0, 0x4431));
    } else {
        // slot t holds k0 + {2t, 2t+1, 8+2t, 9+2t}: elements (k, k+1) -> slot t0,
        // (k+2, k+3) -> slot t0 + 1, bytes 0-1 (r < 8) or 2-3 (r >= 8)
        uint8_t* d = base + half * 4 + ((r & 7) >> 1) * 8 + ((r >> 3) << 1);
        *reinterpret_cast<uint16_t*>(d) = static_cast<uint16_t>(d1);
        *reinterpret_cast<uint16_t*>(d + 8) = static_cast<uint16_t>(d1 >> 16);
        *reinterpret_cast<uint16_t*>(d + 32) = static_cast<uint16_t>(d2);
        *reinterpret_cast<uint16_t*>(d + 40) = static_cast<uint16_t>(d2 >> 16);
        *reinterpret_cast<uint16_t*>(d + 64) = static_cast<uint16_t>(d3);
        *reinterpret_cast<uint16_t*>(d + 72) = static_cast<uint16_t>(d3 >> 16);
    }
}

__host__ __device__ constexpr int gv_jb_for(int M) { return M <= 2 ? 1 : (M <= 5 ? 2 : (M <= 8 ? 3 : 6)); }

// Digits of the whole activation matrix, once per GEMM call with M > 2 (for M <= 2 every
// GEMV CTA makes the digits of its own K-range, which costs less than a launch).  One CTA
// per row: row maximum, power-of-two factor, then the three digit columns of the row in
// the operand order of gemv_mma_kernel.  Rows are served in slabs of 16; slab s owns
// `slab_bytes` of the array, laid out [K/32 blocks][nj columns][32 bytes] with nj = 8 * JB
// of that slab's launch; k >= K is written as zero up to k_pad.
// What the digit pass does to its input before making digits: nothing, RMSNorm of the row
// (src/kernels/normalization.cpp:58-76) or SwiGLU of a [gate || value] row
// (src/kernels/activation.cpp:46-55).  With a prologue the GEMM consumes norm(x) / swiglu(x)
// without that tensor ever being written.
enum GemvPrologue { GV_PRO_NONE = 0, GV_PRO_RMSNORM = 1, GV_PRO_SWIGLU = 2 };

template <int WBITS>
__global__ void __launch_bounds__(1024)
gemv_digits_kernel(const float* __restrict__ A, int M, int K, int k_pad, size_t slab_bytes,
                   uint8_t* __restrict__ digits, float* __restrict__ inv_scale, int prologue,
                   const float* __restrict__ gamma, float eps) {
    __shared__ unsigned s_max[32];
    __shared__ float s_sum[32];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");      // A may come from the kernel before; so may readers of `digits`
    const int row_g = blockIdx.x, slab = row_g / GV_MAX_M, m = row_g % GV_MAX_M;
    const int jb = gv_jb_for(min(GV_MAX_M, M - slab * GV_MAX_M));
    if (jb == 1) return;                                    // a slab of one or two rows makes its own digits
    const int nj = 8 * jb;
    digits += slab * slab_bytes;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t row_len = (prologue == GV_PRO_SWIGLU) ? 2 * static_cast<int64_t>(K) : K;
    const float* row = A + static_cast<int64_t>(row_g) * row_len;
    // Rows of up to 16384 elements stay in registers between the passes (one trip to memory, the
    // prologue computed once); longer rows are re-read and the prologue recomputed.
    constexpr int DC = 4;                                   // float4 per thread held in registers
    const bool cached = K <= 4096 * DC;
    float4 hv[DC];
    if (cached) {
#pragma unroll
        for (int i = 0; i < DC; ++i) {
            const int k = threadIdx.x * 4 + i * 4096;
            hv[i] = (k < K) ? *reinterpret_cast<const float4*>(row + k) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    float inv_rms = 1.0f;
    if (prologue == GV_PRO_RMSNORM) {
        float ss = 0.0f;
        if (cached) {
#pragma unroll
            for (int i = 0; i < DC; ++i) ss += hv[i].x * hv[i].x + hv[i].y * hv[i].y + hv[i].z * hv[i].z + hv[i].w * hv[i].w;
        } else {
            for (int k = threadIdx.x * 4; k < K; k += 4096) {
                const float4 v = *reinterpret_cast<const float4*>(row + k);
                ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
        }
        ss = warp_sum(ss);
        if (lane == 0) s_sum[warp] = ss;
        __syncthreads();
        ss = s_sum[0];
#pragma unroll
        for (int w = 1; w < 32; ++w) ss += s_sum[w];        // same order in every thread
        inv_rms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, static_cast<float>(K)), eps)));
    }
    // the prologue on four consecutive inputs at k (k < K), given their raw values
    auto transform = [&](float4 v, int k) {
        if (prologue == GV_PRO_RMSNORM) {
            const float4 g = *reinterpret_cast<const float4*>(gamma + k);
            v.x = __fmul_rn(__fmul_rn(v.x, inv_rms), g.x); v.y = __fmul_rn(__fmul_rn(v.y, inv_rms), g.y);
            v.z = __fmul_rn(__fmul_rn(v.z, inv_rms), g.z); v.w = __fmul_rn(__fmul_rn(v.w, inv_rms), g.w);
        } else if (prologue == GV_PRO_SWIGLU) {
            const float4 u = *reinterpret_cast<const float4*>(row + K + k);
            v.x = swiglu_one(v.x, u.x); v.y = swiglu_one(v.y, u.y);
            v.z = swiglu_one(v.z, u.z); v.w = swiglu_one(v.w, u.w);
        }
        return v;
    };
    unsigned mxb = 0u;                      // largest magnitude as bits: NaN and Inf survive the maximum
    if (cached) {
#pragma unroll
        for (int i = 0; i < DC; ++i) {
            const int k = threadIdx.x * 4 + i * 4096;
            if (k < K && prologue != GV_PRO_NONE) hv[i] = transform(hv[i], k);
            mxb = max(mxb, abs_bits_max4(hv[i]));
        }
    } else {
        for (int k = threadIdx.x * 4; k < K; k += 4096) {
            const float4 v = transform(*reinterpret_cast<const float4*>(row + k), k);
            mxb = max(mxb, abs_bits_max4(v));
        }
    }
    mxb = __reduce_max_sync(0xffffffffu, mxb);
    if (lane == 0) s_max[warp] = mxb;
    __syncthreads();
    unsigned mb = s_max[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mb = max(mb, __shfl_xor_sync(0xffffffffu, mb, o));
    // power-of-two factor taking max|a| into [2^21, 2^22); exponent clamped
    int se = mb ? 275 - static_cast<int>((mb >> 23) & 0xff) : 127;
    se = max(1, min(253, se));
    const float scl = __uint_as_float(static_cast<uint32_t>(se) << 23);
    if (threadIdx.x == 0) inv_scale[row_g] = digit_inv_scale(mb, se);
    if (cached) {
#pragma unroll
        for (int i = 0; i < DC; ++i) {
            const int k = threadIdx.x * 4 + i * 4096;
            if (k < k_pad) write_digits<WBITS>(digits + (static_cast<int64_t>(k >> 5) * nj + 3 * m) * 32, k & 31, hv[i], scl);
        }
    } else {
        for (int k = threadIdx.x * 4; k < k_pad; k += 4096) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (k < K) v = transform(*reinterpret_cast<const float4*>(row + k), k);
            write_digits<WBITS>(digits + (static_cast<int64_t>(k >> 5) * nj + 3 * m) * 32, k & 31, v, scl);
        }
    }
}

struct GemvParams {
    const float* A;        // [M, K]
    const float* scales;   // W8: [N] (W4 scales arrive through their tensor map)
    float* C;              // [M, N]
    int M, N, K, G;        // G unused for W8
    float alpha, beta;
    int S;                 // stages (units) per column tile = ceil(rows / 64)
    int units;             // column tiles * S
    int nstage;            // ring depth
    int srows;             // W4: scale rows per stage
    int flush_mask;        // W4: bit b set = fold the int32 sums after k32-block b of a stage
    int max_contrib;       // partial slots per column tile in scratch
    float* partial;        // scratch [column tile][max_contrib][M][256]
    int* counters;         // one per column tile, zero between calls
    int* status;
    const uint8_t* digits; // M > 2: activation digits of all of K in operand order, from gemv_digits_kernel
    const float* inv_scale;//        and the inverse of each row's power-of-two factor
    int trace_slot;        // development builds only
};

// WBITS: 4 or 8.  JB: number of 8-column activation blocks; 3 digit columns per
// row of A, so M <= (8 * JB) / 3.
// STAGE_FOLD: W4 with group_size >= 128: the int32 sums are folded exactly once per stage, after
// its last k32-block, so the first block of a stage starts its sums from zero inside the MMA.
// ASYM: asymmetric int4 (W4, group_size 128, STAGE_FOLD): unsigned nibbles, fp16 scale and
// zero-point tiles (tmS, tmZ), and per stage  sum_k a_k (u_k - z) = sum_k a_k u_k - z * sum_k a_k,
// the second term from per-stage sums of the activation digits.
template <int WBITS, int JB, bool STAGE_FOLD, bool ASYM>
__global__ void __launch_bounds__(gv_threads(JB), (JB >= 6) ? 1 : 2)
gemv_mma_kernel(const __grid_constant__ TensorMap tmB, const __grid_constant__ TensorMap tmS,
                const __grid_constant__ TensorMap tmZ, const GemvParams p) {
    constexpr int K_PER_ROW = (WBITS == 4) ? 2 : 1;
    constexpr int KPS = GV_ROWS * K_PER_ROW;              // k per stage: 128 (W4), 64 (W8)
    constexpr int KPS_SHIFT = (WBITS == 4) ? 7 : 6;
    constexpr int KB = KPS / 32;                          // k32 blocks per stage: 4 (W4), 2 (W8)
    constexpr int NJ = 8 * JB;                            // digit columns
    constexpr int GV_CONSUMER_WARPS = gv_consumer_warps(JB);
    constexpr int GV_CONSUMERS = GV_CONSUMER_WARPS * 32;
    constexpr int GV_THREADS = gv_threads(JB);
    constexpr int JBL = JB / gv_groups(JB);               // digit blocks of one consumer warp

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int NST = p.nstage;
    uint8_t* tiles = smem;                                             // NST * 16 KiB
    float* sc = reinterpret_cast<float*>(smem + NST * GV_STAGE_BYTES);            // W4: [NST][srows][256]
    float* part = sc + NST * p.srows * GV_COLS;                        // [NJ][256]
    float* inv_s = part + NJ * GV_COLS;                                // [16]
    unsigned* rowmax = reinterpret_cast<unsigned*>(inv_s + 16);        // [16] max|a| bits per row
    uint64_t* bars = reinterpret_cast<uint64_t*>(rowmax + 16);         // full[], empty[]
    int* flags = reinterpret_cast<int*>(bars + 2 * GV_MAX_STAGE + 2);  // after the digit barrier; [0] abort, [1] is-last
    uint8_t* dfrag = reinterpret_cast<uint8_t*>(flags + 4);            // [digit stage][kb32][NJ][32]
    volatile int* abort_flag = flags;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int S = p.S;
    GV_STAMP(0);
    const int u0 = static_cast<int>(static_cast<int64_t>(blockIdx.x) * p.units / gridDim.x);
    const int u1 = static_cast<int>(static_cast<int64_t>(blockIdx.x + 1) * p.units / gridDim.x);
    const int n_units = u1 - u0;
    const int tile_first = u0 / S;
    const int s_first = u0 - tile_first * S;
    const int n_dig = min(S, n_units);                     // distinct stages of K this CTA meets

    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + GV_MAX_STAGE);
    const uint32_t digbar = smem_u32(bars + 2 * GV_MAX_STAGE);        // M > 2: the digits have landed
    const uint32_t stage_tx = GV_STAGE_BYTES + ((WBITS == 4) ? p.srows * GV_COLS * 4 : 0);
    // one unit into ring slot `slot`: two weight boxes and, for W4, its rows of group scales
    auto issue = [&](int tile, int stage, int slot) {
        const uint32_t bar = full0 + 8 * slot;
        ptx::mbar_expect_tx(bar, stage_tx);
#pragma unroll
        for (int b = 0; b < GV_BOXES; ++b)
            ptx::tma_load_2d(smem_u32(tiles + slot * GV_STAGE_BYTES + b * GV_BOX_BYTES), &tmB,
                             tile * GV_COLS + b * GV_BOX_COLS, stage * GV_ROWS, bar);
        if (ASYM) {
            // one group per stage: 256 fp16 scales, then 256 fp16 zero-points, in the stage's 1 KiB
            ptx::tma_load_2d(smem_u32(sc + slot * GV_COLS), &tmS, tile * GV_COLS, stage, bar);
            ptx::tma_load_2d(smem_u32(sc + slot * GV_COLS) + GV_COLS * 2, &tmZ, tile * GV_COLS, stage, bar);
        } else if (WBITS == 4) {
            const int row = (p.G >= KPS) ? (stage * KPS) / p.G : stage * p.srows;
            ptx::tma_load_2d(smem_u32(sc + slot * p.srows * GV_COLS), &tmS, tile * GV_COLS, row, bar);
        }
    };
    // The producer thread sets the barriers up and puts the first ring-full of units
    // in flight before anything else happens in the CTA.
    int prod_tile = tile_first, prod_stage = s_first;
    if (warp == GV_CONSUMER_WARPS && lane == 0) {
        for (int s = 0; s < GV_MAX_STAGE; ++s) {
            ptx::mbar_init(full0 + 8 * s, 1);
            ptx::mbar_init(empty0 + 8 * s, GV_CONSUMER_WARPS);
        }
        ptx::mbar_init(digbar, 1);
        flags[0] = 0;
        flags[1] = 0;
        ptx::fence_mbar_init();
        const int first = min(n_units, NST);
        for (int s = 0; s < first; ++s) {
            issue(prod_tile, prod_stage, s);
            if (++prod_stage == S) { prod_stage = 0; ++prod_tile; }
        }
    }
    if (threadIdx.x < 16) rowmax[threadIdx.x] = 0u;
    // Programmatic dependent launch: the weight loads above depend on nothing an
    // earlier kernel in the stream writes, so they are already in flight while
    // that kernel drains; everything below (activations, C, scratch, counters)
    // waits for it to finish.  The next kernel may be scheduled from here on.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    GV_STAMP(1);
    __syncthreads();

    // ---- prologue, overlapped with the loads in flight ---------------------------
    constexpr bool PRE = JB > 1;        // digits were made once for all CTAs by gemv_digits_kernel
    if constexpr (PRE) {
        // digit stage i = stage (s_first + i) mod S: one or two contiguous pieces of the global array
        if (warp == GV_CONSUMER_WARPS && lane == 0) {
            const uint32_t per_stage = KPS * NJ;
            const int len_a = min(n_dig, S - s_first);
            ptx::mbar_expect_tx(digbar, n_dig * per_stage);
            ptx::bulk_load_1d(smem_u32(dfrag), p.digits + static_cast<int64_t>(s_first) * per_stage, len_a * per_stage,
                              digbar);
            if (n_dig > len_a)
                ptx::bulk_load_1d(smem_u32(dfrag) + len_a * per_stage, p.digits, (n_dig - len_a) * per_stage, digbar);
        }
        if (threadIdx.x < p.M) inv_s[threadIdx.x] = p.inv_scale[threadIdx.x];
        ptx::mbar_wait(digbar, 0, abort_flag, p.status);
        __syncthreads();
    } else {
    // Activations of the K stages this CTA meets (digit stage i = stage
    // (s_first + i) mod S): row maxima, then three 8-bit digits per element in
    // MMA-operand order.  Digit columns of rows m >= M are left as they are: an
    // MMA column only feeds its own output column, never read.
    const int q4 = n_dig * (KPS / 4);                      // float4 per row
    const int n4 = p.M * q4;
    const int n4_pad = (n4 + 31) & ~31;                    // whole warps take part in the shuffles
    const float inv_q4 = 1.0f / static_cast<float>(q4 > 0 ? q4 : 1);
    // global k of local element kl (a multiple of 4) of the digit stages
    auto k_of = [&](int kl) {
        int stage = s_first + (kl >> KPS_SHIFT);
        if (stage >= S) stage -= S;
        return stage * KPS + (kl & (KPS - 1));
    };
    // Loads are issued GV_PB at a time per thread before any of them is used: the
    // prologue's cost is a few memory round trips, not one per float4.
    for (int base = 0; base < n4_pad; base += GV_PB * GV_THREADS) {
        float4 v[GV_PB];
        int mrow[GV_PB];
#pragma unroll
        for (int j = 0; j < GV_PB; ++j) {
            const int i = base + j * GV_THREADS + threadIdx.x;
            // row index without an integer division: (i + 0.5) / q4 is never within
            // 0.5 / q4 of an integer, far more than the float error at these sizes
            const int m = (i < n4) ? min(p.M - 1, __float2int_rz((static_cast<float>(i) + 0.5f) * inv_q4)) : -1;
            mrow[j] = m;
            v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (m >= 0) {
                const int k = k_of((i - m * q4) * 4);
                if (k < p.K) v[j] = *reinterpret_cast<const float4*>(p.A + static_cast<int64_t>(m) * p.K + k);
            }
        }
#pragma unroll
        for (int j = 0; j < GV_PB; ++j) {
            if (base + j * GV_THREADS + (threadIdx.x & ~31) >= n4_pad) break;      // warp-uniform
            const int m = mrow[j];
            unsigned mx = abs_bits_max4(v[j]);             // as bits: a NaN or an infinity wins the maximum
            const int m0 = __shfl_sync(0xffffffffu, m, 0);
            if (__all_sync(0xffffffffu, m == m0)) {        // the usual case: one row per warp step
                mx = __reduce_max_sync(0xffffffffu, mx);
                if (lane == 0 && m0 >= 0 && mx > 0u) atomicMax(rowmax + m0, mx);
            } else if (m >= 0 && mx > 0u) {
                atomicMax(rowmax + m, mx);
            }
        }
    }
    __syncthreads();
    for (int base = 0; base < n4; base += GV_PB * GV_THREADS) {
      float4 vb[GV_PB];
#pragma unroll
      for (int j = 0; j < GV_PB; ++j) {
          const int i = base + j * GV_THREADS + threadIdx.x;
          vb[j] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (i < n4) {
              const int m = min(p.M - 1, __float2int_rz((static_cast<float>(i) + 0.5f) * inv_q4));
              const int k = k_of((i - m * q4) * 4);
              if (k < p.K) vb[j] = *reinterpret_cast<const float4*>(p.A + static_cast<int64_t>(m) * p.K + k);
          }
      }
#pragma unroll
      for (int j = 0; j < GV_PB; ++j) {
        const int i = base + j * GV_THREADS + threadIdx.x;
        if (i >= n4) break;
        const int m = min(p.M - 1, __float2int_rz((static_cast<float>(i) + 0.5f) * inv_q4));
        const int kl = (i - m * q4) * 4;
        // power-of-two factor taking max|a| into [2^21, 2^22); exponent clamped
        const unsigned mb = rowmax[m];
        int se = mb ? 275 - static_cast<int>((mb >> 23) & 0xff) : 127;     // 127 + 21 - (e - 127)
        se = max(1, min(253, se));
        const float scl = __uint_as_float(static_cast<uint32_t>(se) << 23);
        if (kl == 0) inv_s[m] = digit_inv_scale(mb, se);
        const float4 v = vb[j];
        write_digits<WBITS>(dfrag + ((kl >> 5) * NJ + 3 * m) * 32, kl & 31, v, scl);
      }
    }
    __syncthreads();
    }   // !PRE
    // ASYM: sum of each digit column over each digit stage (= one quantisation group)
    float* dsum = reinterpret_cast<float*>(dfrag + n_dig * (KPS * NJ));       // [digit stage][NJ]
    if constexpr (ASYM) {
        for (int i = threadIdx.x; i < n_dig * NJ; i += GV_THREADS) {
            const int ds_i = i / NJ, j = i - ds_i * NJ;
            int sum = 0;
#pragma unroll
            for (int kb = 0; kb < KB; ++kb) {
                const uint32_t* w = reinterpret_cast<const uint32_t*>(dfrag + ((ds_i * KB + kb) * NJ + j) * 32);
#pragma unroll
                for (int q = 0; q < 8; ++q) sum = __dp4a(static_cast<int>(w[q]), 0x01010101, sum);
            }
            dsum[i] = static_cast<float>(sum);
        }
        __syncthreads();
    }
    GV_STAMP(2);

    if (warp < GV_CONSUMER_WARPS) {
        // A warp owns two 16-column fragments f = 0, 1: columns 32*cw + 16*f .. +15 of the
        // tile (cw = its column-warp index), i.e. 16-byte chunks 2*(cw%4) + f of box cw/4,
        // and the digit blocks jb0 .. jb0 + JBL - 1 of its group.
        const int g = lane >> 2, t = lane & 3;
        const int cw = warp & (GV_COL_WARPS - 1), jb0 = (warp / GV_COL_WARPS) * JBL;
        const int box = cw >> 2, chunk0 = (cw & 3) * 2;
        const int wcol = cw * 32 + 2 * g;                   // + 16*f: this thread's column pair in the tile
        const int lrow = lane & 7, lmat = lane >> 3;
        // ldmatrix source of this lane inside a stage, per half (32 byte-rows) and fragment
        uint32_t ldoff[2][2];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int row = half * 32 + lmat * 8 + lrow;
#pragma unroll
            for (int f = 0; f < 2; ++f)
                ldoff[half][f] = box * GV_BOX_BYTES + row * 128 + (((chunk0 + f) ^ (row & 7)) << 4);
        }
        const uint8_t* dlane = dfrag + (jb0 * 8 + g) * 32 + t * 8;     // + ((digit stage * KB + kb) * NJ + jb * 8) * 32
        const uint32_t tiles0 = smem_u32(tiles);

        float out[2][JBL][4];
        int acc[2][JBL][4];
        auto clear = [&]() {
#pragma unroll
            for (int f = 0; f < 2; ++f)
#pragma unroll
                for (int jb = 0; jb < JBL; ++jb)
#pragma unroll
                    for (int i = 0; i < 4; ++i) { out[f][jb][i] = 0.0f; acc[f][jb][i] = 0; }
        };
        // fold the int32 sums into fp32, times the scales at `srow` (W4) or 1 (W8)
        auto flush_asym = [&](const float* stile, const float* dsum_stage) {
            // stile: 256 fp16 scales, then 256 fp16 zero-points of this stage's group
            const __half* sh = reinterpret_cast<const __half*>(stile);
#pragma unroll
            for (int f = 0; f < 2; ++f) {
                const float2 sv = __half22float2(*reinterpret_cast<const __half2*>(sh + wcol + 16 * f));
                const float2 zv = __half22float2(*reinterpret_cast<const __half2*>(sh + GV_COLS + wcol + 16 * f));
                const float z0 = -16.0f * zv.x, z1 = -16.0f * zv.y;      // weights are carried as 16 * u
#pragma unroll
                for (int jb = 0; jb < JBL; ++jb) {
                    const float2 sd = *reinterpret_cast<const float2*>(dsum_stage + (jb0 + jb) * 8 + 2 * t);
                    out[f][jb][0] = fmaf(sv.x, fmaf(z0, sd.x, small_int_to_float(acc[f][jb][0])), out[f][jb][0]);
                    out[f][jb][1] = fmaf(sv.x, fmaf(z0, sd.y, small_int_to_float(acc[f][jb][1])), out[f][jb][1]);
                    out[f][jb][2] = fmaf(sv.y, fmaf(z1, sd.x, small_int_to_float(acc[f][jb][2])), out[f][jb][2]);
                    out[f][jb][3] = fmaf(sv.y, fmaf(z1, sd.y, small_int_to_float(acc[f][jb][3])), out[f][jb][3]);
                }
            }
        };
        auto flush = [&](const float* srow) {
#pragma unroll
            for (int f = 0; f < 2; ++f) {
                float s0 = 1.0f, s1 = 1.0f;
                if (WBITS == 4) {
                    const float2 sv = *reinterpret_cast<const float2*>(srow + wcol + 16 * f);
                    s0 = sv.x; s1 = sv.y;
                }
#pragma unroll
                for (int jb = 0; jb < JBL; ++jb) {
                    out[f][jb][0] = fmaf(s0, small_int_to_float(acc[f][jb][0]), out[f][jb][0]);
                    out[f][jb][1] = fmaf(s0, small_int_to_float(acc[f][jb][1]), out[f][jb][1]);
                    out[f][jb][2] = fmaf(s1, small_int_to_float(acc[f][jb][2]), out[f][jb][2]);
                    out[f][jb][3] = fmaf(s1, small_int_to_float(acc[f][jb][3]), out[f][jb][3]);
                    if (!STAGE_FOLD) acc[f][jb][0] = acc[f][jb][1] = acc[f][jb][2] = acc[f][jb][3] = 0;
                }
            }
        };
        // one k32-block: the activation fragment is loaded once and feeds both column fragments
        auto mma_block = [&](const uint8_t* dblk, const uint32_t (&a)[2][4], bool first) {
#pragma unroll
            for (int jb = 0; jb < JBL; ++jb) {
                const uint2 b = *reinterpret_cast<const uint2*>(dblk + jb * 8 * 32);
                if (ASYM) {
                    if (first) {
                        mma_u8s8_16832_first(acc[0][jb], a[0][0], a[0][1], a[0][2], a[0][3], b.x, b.y);
                        mma_u8s8_16832_first(acc[1][jb], a[1][0], a[1][1], a[1][2], a[1][3], b.x, b.y);
                    } else {
                        mma_u8s8_16832(acc[0][jb], a[0][0], a[0][1], a[0][2], a[0][3], b.x, b.y);
                        mma_u8s8_16832(acc[1][jb], a[1][0], a[1][1], a[1][2], a[1][3], b.x, b.y);
                    }
                } else if (first) {
                    mma_s8_16832_first(acc[0][jb], a[0][0], a[0][1], a[0][2], a[0][3], b.x, b.y);
                    mma_s8_16832_first(acc[1][jb], a[1][0], a[1][1], a[1][2], a[1][3], b.x, b.y);
                } else {
                    mma_s8_16832(acc[0][jb], a[0][0], a[0][1], a[0][2], a[0][3], b.x, b.y);
                    mma_s8_16832(acc[1][jb], a[1][0], a[1][1], a[1][2], a[1][3], b.x, b.y);
                }
            }
        };

        int slot = 0, didx = 0;
        uint32_t phase = 0;
        int u = u0;
        int tile = tile_first, s_begin = s_first;
        while (u < u1) {
            const int s_end = min(S, s_begin + (u1 - u));
            clear();
            int unflushed = 0;                              // W8: stages since the last fold
            for (int s = s_begin; s < s_end; ++s) {
                const bool ok = ptx::mbar_wait(full0 + 8 * slot, phase, abort_flag, p.status);
                const uint32_t tile_s = tiles0 + slot * GV_STAGE_BYTES;
                const uint8_t* dst = dlane + didx * (KB * NJ * 32);
                const float* sstage = sc + slot * p.srows * GV_COLS;
                if (ok) {
                    int srow_i = 0;
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        // register x[f][j]: bytes {row 2t: col 2g, col 2g+1; row 2t+1: col 2g, col 2g+1}
                        // of byte-rows 8j .. 8j+7 of this 32-row half, fragment f
                        uint32_t x[2][4];
                        ldmatrix_x4_trans(tile_s + ldoff[half][0], x[0]);
                        ldmatrix_x4_trans(tile_s + ldoff[half][1], x[1]);
                        if (WBITS == 4) {
#pragma unroll
                            for (int q = 0; q < 2; ++q) {           // k32-block 2*half + q: matrices 2q, 2q+1
                                uint32_t a[2][4];
#pragma unroll
                                for (int f = 0; f < 2; ++f) {
                                    // four byte-rows {2t, 2t+1, 8+2t, 9+2t} of column 2g / 2g+1
                                    const uint32_t e0 = __byte_perm(x[f][2 * q], x[f][2 * q + 1], 0x6420);
                                    const uint32_t e1 = __byte_perm(x[f][2 * q], x[f][2 * q + 1], 0x7531);
                                    a[f][0] = (e0 << 4) & 0xf0f0f0f0u;     // even k, int8 = 16*q
                                    a[f][1] = (e1 << 4) & 0xf0f0f0f0u;
                                    a[f][2] = e0 & 0xf0f0f0f0u;            // odd k
                                    a[f][3] = e1 & 0xf0f0f0f0u;
                                }
                                const int kb = 2 * half + q;
                                mma_block(dst + kb * NJ * 32, a, STAGE_FOLD && kb == 0);
                                if (STAGE_FOLD) {
                                    if (kb == KB - 1) {
                                        if (ASYM) flush_asym(sstage, dsum + didx * NJ);
                                        else flush(sstage);
                                    }
                                } else if (p.flush_mask & (1 << kb)) {
                                    flush(sstage + srow_i * GV_COLS);
                                    ++srow_i;
                                }
                            }
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
                            mma_block(dst + half * NJ * 32, a, false);
                        }
                    }
                    if (WBITS == 8 && ++unflushed == 4) { unflushed = 0; flush(nullptr); }
                }
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(empty0 + 8 * slot);      // stage (weights and scales) fully read
                if (++slot == NST) { slot = 0; phase ^= 1; }
                if (++didx == n_dig) didx = 0;
            }
            if (WBITS == 8 && unflushed != 0) flush(nullptr);
            GV_STAMP(3);

            // ---- end of a segment: digit columns -> [M, 256] tile ----
            // per-column partial sums: column j of the operand = digit (j % 3) of row j / 3.
            // M > 2: through shared memory.  M <= 2: the three digits of a row sit in two
            // neighbouring lanes, so a shuffle brings them together (further down).
            if constexpr (JB > 1) {
#pragma unroll
            for (int f = 0; f < 2; ++f) {
                float c0 = 1.0f, c1 = 1.0f;
                if (WBITS == 8) {
                    const int n_a = tile * GV_COLS + wcol + 16 * f;
                    c0 = (n_a < p.N) ? p.scales[n_a] : 0.0f;
                    c1 = (n_a + 1 < p.N) ? p.scales[n_a + 1] : 0.0f;
                }
#pragma unroll
                for (int jb = 0; jb < JBL; ++jb) {
                    float* d = part + ((jb0 + jb) * 8 + 2 * t) * GV_COLS + wcol + 16 * f;
                    *reinterpret_cast<float2*>(d) = make_float2(c0 * out[f][jb][0], c1 * out[f][jb][2]);
                    *reinterpret_cast<float2*>(d + GV_COLS) = make_float2(c0 * out[f][jb][1], c1 * out[f][jb][3]);
                }
            }
            consumer_sync<GV_CONSUMERS>();
            }

            const bool whole = (s_begin == 0 && s_end == S);       // this segment is all of K
            const int col0 = tile * GV_COLS;
            const int ncol = min(GV_COLS, p.N - col0);             // multiple of 16
            const float digit_unit = (WBITS == 4) ? 0.0625f : 1.0f;     // int4 nibbles were carried as 16*q
            // contributors to this column tile are the CTAs cf..cl; contributor i owns partial slot i
            int cf = 0, n_contrib = 1;
            if (!whole) {
                const int64_t P = gridDim.x;
                cf = static_cast<int>(((static_cast<int64_t>(tile) * S + 1) * P - 1) / p.units);
                const int cl = static_cast<int>(((static_cast<int64_t>(tile + 1) * S) * P - 1) / p.units);
                n_contrib = cl - cf + 1;
            }
            float* slot_base = p.partial + (static_cast<int64_t>(tile) * p.max_contrib) * p.M * GV_COLS;
            float* my_slot = slot_base + static_cast<int64_t>(blockIdx.x - cf) * p.M * GV_COLS;
            auto store_c = [&](int m, int c, float4 v) {
                float4* cp = reinterpret_cast<float4*>(p.C + static_cast<int64_t>(m) * p.N + col0 + c);
                if (p.beta == 0.0f) {
                    v.x *= p.alpha; v.y *= p.alpha; v.z *= p.alpha; v.w *= p.alpha;
                } else {
                    const float4 o = *cp;
                    v.x = fmaf(p.beta, o.x, p.alpha * v.x); v.y = fmaf(p.beta, o.y, p.alpha * v.y);
                    v.z = fmaf(p.beta, o.z, p.alpha * v.z); v.w = fmaf(p.beta, o.w, p.alpha * v.w);
                }
                *cp = v;
            };
            if constexpr (JB == 1) {
                // lane t = 0 holds digits 0, 1 of row 0 and gets digit 2 from lane t = 1; lane t = 2
                // holds digits 1, 2 of row 1 (operand columns 4, 5) and gets digit 0 (column 3)
                // from lane t = 1.  Values: out[f][0][{0,1}] = column wcol, digit columns 2t, 2t+1;
                // out[f][0][{2,3}] = column wcol + 1.
#pragma unroll
                for (int f = 0; f < 2; ++f) {
                    float c0 = 1.0f, c1 = 1.0f;
                    const int cc = wcol + 16 * f;
                    if (WBITS == 8) {
                        c0 = (col0 + cc < p.N) ? p.scales[col0 + cc] : 0.0f;
                        c1 = (col0 + cc + 1 < p.N) ? p.scales[col0 + cc + 1] : 0.0f;
                    }
                    const float e0 = out[f][0][0], o0 = out[f][0][1], e1 = out[f][0][2], o1 = out[f][0][3];
                    const float up_e0 = __shfl_down_sync(0xffffffffu, e0, 1), up_e1 = __shfl_down_sync(0xffffffffu, e1, 1);
                    const float dn_o0 = __shfl_up_sync(0xffffffffu, o0, 1), dn_o1 = __shfl_up_sync(0xffffffffu, o1, 1);
                    const int m = t >> 1;                          // t = 0 -> row 0, t = 2 -> row 1
                    if ((t & 1) == 0 && m < p.M && cc < ncol) {
                        const float is = inv_s[m] * digit_unit;
                        float2 v;
                        if (t == 0) {
                            v.x = c0 * is * fmaf(65536.0f, e0, fmaf(256.0f, o0, up_e0));
                            v.y = c1 * is * fmaf(65536.0f, e1, fmaf(256.0f, o1, up_e1));
                        } else {
                            v.x = c0 * is * fmaf(65536.0f, dn_o0, fmaf(256.0f, e0, o0));
                            v.y = c1 * is * fmaf(65536.0f, dn_o1, fmaf(256.0f, e1, o1));
                        }
                        if (whole) {
                            float2* cp = reinterpret_cast<float2*>(p.C + static_cast<int64_t>(m) * p.N + col0 + cc);
                            if (p.beta == 0.0f) {
                                v.x *= p.alpha; v.y *= p.alpha;
                            } else {
                                const float2 o = *cp;
                                v.x = fmaf(p.beta, o.x, p.alpha * v.x); v.y = fmaf(p.beta, o.y, p.alpha * v.y);
                            }
                            *cp = v;
                        } else {
                            *reinterpret_cast<float2*>(my_slot + m * GV_COLS + cc) = v;
                        }
                    }
                }
            } else
            for (int i = threadIdx.x; i < p.M * (GV_COLS / 4); i += GV_CONSUMERS) {
                const int m = i >> 6, c = (i & 63) * 4;
                if (c >= ncol) continue;
                const float4 h = *reinterpret_cast<const float4*>(part + (3 * m) * GV_COLS + c);
                const float4 md = *reinterpret_cast<const float4*>(part + (3 * m + 1) * GV_COLS + c);
                const float4 l = *reinterpret_cast<const float4*>(part + (3 * m + 2) * GV_COLS + c);
                const float is = inv_s[m] * digit_unit;
                float4 v;
                v.x = is * fmaf(65536.0f, h.x, fmaf(256.0f, md.x, l.x));
                v.y = is * fmaf(65536.0f, h.y, fmaf(256.0f, md.y, l.y));
                v.z = is * fmaf(65536.0f, h.z, fmaf(256.0f, md.z, l.z));
                v.w = is * fmaf(65536.0f, h.w, fmaf(256.0f, md.w, l.w));
                if (whole) store_c(m, c, v);
                else *reinterpret_cast<float4*>(my_slot + m * GV_COLS + c) = v;
            }
            if (!whole) {
                // the last contributor to arrive sums the partials in contributor order and writes C
                consumer_sync<GV_CONSUMERS>();
                GV_STAMP(4);
                // One thread fences for the CTA on either side of the count (a fence per thread
                // costs microseconds here): the barrier before orders every consumer's partial
                // stores ahead of it, the barrier after orders the other contributors' stores
                // ahead of every consumer's loads.
                if (threadIdx.x == 0) {
                    __threadfence();
                    const int old = atomicAdd(p.counters + tile, 1);
                    flags[1] = (old == n_contrib - 1);
                    if (old == n_contrib - 1) {
                        p.counters[tile] = 0;                          // ready for the next call
                        __threadfence();                               // only the summing CTA reads the others' stores
                    }
                }
                consumer_sync<GV_CONSUMERS>();
                GV_STAMP(5);
                if (flags[1]) {
                    for (int i = threadIdx.x; i < p.M * (GV_COLS / 4); i += GV_CONSUMERS) {
                        const int m = i >> 6, c = (i & 63) * 4;
                        if (c >= ncol) continue;
                        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
                        // eight partials in flight at a time: one memory round trip per eight
                        // contributors, summed in contributor order
                        for (int r0 = 0; r0 < n_contrib; r0 += 8) {
                            float4 v[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j)         // unconditional (clamped) so that they overlap
                                v[j] = __ldcg(reinterpret_cast<const float4*>(
                                    slot_base + (static_cast<int64_t>(min(r0 + j, n_contrib - 1)) * p.M + m) * GV_COLS + c));
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                if (r0 + j < n_contrib) { sum.x += v[j].x; sum.y += v[j].y; sum.z += v[j].z; sum.w += v[j].w; }
                        }
                        store_c(m, c, sum);
                    }
                }
            }
            consumer_sync<GV_CONSUMERS>();                                // `part` and flags[1] are free again
            GV_STAMP(6);
            u += s_end - s_begin;
            s_begin = 0;
            ++tile;
        }
    } else if (lane == 0) {
        // producer: refill ring slots as the consumers release them
        int issued = min(n_units, NST);
        int slot = 0;
        uint32_t phase = 0;                                // parity of the consumers' release being waited for
        for (int ui = NST; ui < n_units; ++ui) {
            if (!ptx::mbar_wait(empty0 + 8 * slot, phase, abort_flag, p.status)) break;
            issue(prod_tile, prod_stage, slot);
            if (++prod_stage == S) { prod_stage = 0; ++prod_tile; }
            issued = ui + 1;
            if (++slot == NST) { slot = 0; phase ^= 1; }
        }
        if (*abort_flag) {
            // a wait ran out: let the copies still in flight land before the CTA exits
            for (int ui = max(0, issued - NST); ui < issued; ++ui) {
                const uint64_t t0 = ptx::global_timer_ns();
                while (!ptx::mbar_try_wait(full0 + 8 * (ui % NST), (ui / NST) & 1))
                    if (ptx::global_timer_ns() - t0 > 200000000ull) break;
            }
        }
    }
}

// ---- host side --------------------------------------------------------------------

struct GemvPlan {
    int S, col_tiles, units, ctas, nstage, srows, flush_mask, max_contrib;
    size_t smem;
    bool ok;
};

static bool w4_group_ok(int G) { return G == 32 || G == 64 || (G >= 128 && G % 128 == 0); }

// Split the units over the CTAs.  The grid is one full wave of the CTAs the SMs can
// hold (two per SM up to M = 8, one for M <= 16) unless a CTA's share of K needs
// more shared memory for its activation digits than there is; then there are more,
// smaller CTAs.  The ring takes what shared memory remains, up to GV_MAX_STAGE.
static GemvPlan plan_gemv(int wbits, int jb, int N, int K, int G, int sm_count, bool asym = false) {
    GemvPlan pl{};
    const int kps = GV_ROWS * (wbits == 4 ? 2 : 1);
    pl.S = ceil_div(K, kps);
    pl.col_tiles = ceil_div(N, GV_COLS);
    const int64_t units = static_cast<int64_t>(pl.S) * pl.col_tiles;
    if (units <= 0 || units > (1 << 30)) return pl;
    pl.units = static_cast<int>(units);
    pl.srows = wbits == 4 ? (G < 128 ? 128 / G : 1) : 0;
    pl.flush_mask = wbits == 4 ? (G == 32 ? 0xF : (G == 64 ? 0xA : 0x8)) : 0;
    int per_sm = jb >= 6 ? 1 : 2;                          // what the kernel's launch bounds allow
    if (knobs().gemv_ctas_per_sm > 0) per_sm = std::min(per_sm, knobs().gemv_ctas_per_sm);
    const size_t nj = 8 * jb;
    const size_t stage_bytes = GV_STAGE_BYTES + static_cast<size_t>(pl.srows) * GV_COLS * 4;
    const size_t fixed = 1024 + nj * GV_COLS * 4 + 16 * 4 + 16 * 4 + (2 * GV_MAX_STAGE + 2) * 8 + 16;
    const size_t dig_per_stage = static_cast<size_t>(kps) * nj + (asym ? nj * 4 : 0);   // digits (+ their sums)
    // Measured on B200: leaving part of the SM's 228 KiB to the L1 cache pays - a lone CTA per SM runs the
    // 16-row int8 shape in 15.0 us with 160 KiB against 16.1 us with everything, and two CTAs per SM run the
    // one-row shape in 10.9 us with four stages each against 11.1 us with five and 11.0 us with three (cap below).
    size_t budget = per_sm == 1 ? 160 * 1024 : (228 * 1024) / per_sm - 1024 - 512;
    if (knobs().gemv_smem_kb > 0) budget = std::min<size_t>(budget, static_cast<size_t>(knobs().gemv_smem_kb) * 1024);
    int ctas = static_cast<int>(std::min<int64_t>(units, static_cast<int64_t>(per_sm) * sm_count));
    // with fewer column tiles than CTAs, a whole number of CTAs per tile: no CTA then
    // straddles two tiles and pays for two hand-offs
    if (pl.col_tiles <= ctas) ctas = pl.col_tiles * std::min(pl.S, ctas / pl.col_tiles);
    int range = ceil_div(pl.units, ctas);
    if (fixed + 2 * stage_bytes + dig_per_stage * std::min(pl.S, range) > budget) {
        // digits of a whole range do not fit: shorter ranges, more CTAs
        if (fixed + 2 * stage_bytes + dig_per_stage > budget) return pl;
        const int r_max = static_cast<int>((budget - fixed - 2 * stage_bytes) / dig_per_stage);
        ctas = ceil_div(pl.units, r_max);
        // more CTAs than the device holds at once: whole waves of equal ranges, so that the
        // last wave is not a handful of CTAs with everybody else idle
        const int capacity = per_sm * sm_count;
        if (ctas > capacity) ctas = static_cast<int>(std::min<int64_t>(units, static_cast<int64_t>(ceil_div(ctas, capacity)) * capacity));
        else if (pl.col_tiles <= ctas && pl.col_tiles * ceil_div(ctas, pl.col_tiles) <= capacity)
            ctas = pl.col_tiles * ceil_div(ctas, pl.col_tiles);
        range = ceil_div(pl.units, ctas);
    }
    const size_t dig = dig_per_stage * std::min(pl.S, range);
    pl.ctas = ctas;
    pl.nstage = static_cast<int>(std::min<size_t>(GV_MAX_STAGE, (budget - fixed - dig) / stage_bytes));
    if (per_sm == 2 && jb == 1) pl.nstage = std::min(pl.nstage, 4);
    pl.nstage = std::max(2, std::min(pl.nstage, std::max(2, range)));
    pl.smem = fixed + dig + pl.nstage * stage_bytes;
    const int r_min = std::max(1, pl.units / ctas);
    pl.max_contrib = std::min(ctas, pl.S / r_min + 2);
    pl.ok = true;
    return pl;
}

static int jb_for(int M) { return gv_jb_for(M); }

bool w4a16_fast_ok(int M, int N, int K, int G) {
    if (M < 1 || (N % 16) != 0 || (K % 32) != 0 || G <= 0 || (K % G) != 0) return false;
    if (!w4_group_ok(G)) return false;            // groups must tile a 128-k stage, or be whole stages
    if (M > 1024) return false;                   // rows are served in slabs of 16; beyond this the generic kernel
    if (M > 2 && static_cast<size_t>(ceil_div(K, 128) * 128) * 48 > GV_DIG_BYTES - GV_INV_BYTES) return false;
    return plan_gemv(4, jb_for(std::min(M, GV_MAX_M)), N, K, G, 148).ok;
}

bool w8a16_fast_ok(int M, int N, int K) {
    if (M < 1 || (N % 16) != 0 || (K % 32) != 0) return false;
    if (M > 1024) return false;
    if (M > 2 && static_cast<size_t>(ceil_div(K, 64) * 64) * 48 > GV_DIG_BYTES - GV_INV_BYTES) return false;
    return plan_gemv(8, jb_for(std::min(M, GV_MAX_M)), N, K, 1, 148).ok;
}

template <int WBITS, int JB, bool STAGE_FOLD, bool ASYM = false>
static int launch_gemv_t(lhb_ctx* ctx, const TensorMap& tm, const TensorMap& tms, const TensorMap& tmz, GemvParams p,
                         const GemvPlan& pl, cudaStream_t st) {
    auto kern = gemv_mma_kernel<WBITS, JB, STAGE_FOLD, ASYM>;
    static bool attr_set[64] = {};                // per instantiation and device
    if (!attr_set[ctx->device & 63]) {
        LHB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        attr_set[ctx->device & 63] = true;
    }
    p.S = pl.S;
    p.units = pl.units;
    p.nstage = pl.nstage;
    p.srows = pl.srows;
    p.flush_mask = pl.flush_mask;
    p.max_contrib = pl.max_contrib;
    p.partial = reinterpret_cast<float*>(static_cast<uint8_t*>(ctx->scratch) + GV_DIG_BYTES);
    p.counters = ctx->counters;
    p.status = ctx->status_word;
#ifdef LHB_GEMV_TRACE
    static int trace_calls = 0;
    p.trace_slot = (trace_calls++) & 63;
#endif
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(pl.ctas, 1, 1);
    cfg.blockDim = dim3(gv_threads(JB), 1, 1);
    cfg.dynamicSmemBytes = pl.smem;
    cfg.stream = st;
    const bool pdl = knobs().pdl;
    cudaLaunchAttribute attr[1];
    int na = 0;
    if (pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    LHB_CUDA(cudaLaunchKernelEx(&cfg, kern, tm, tms, tmz, p));
    return LHB_OK;
}

template <int WBITS, bool ASYM = false>
static int launch_gemv(lhb_ctx* ctx, const float* A, const void* B, const void* scales_v, const void* zeros, float* C,
                       int M, int N, int K, int G, float alpha, float beta, cudaStream_t st,
                       int prologue = GV_PRO_NONE, const float* gamma = nullptr, float eps = 0.0f) {
    const float* scales = ASYM ? nullptr : static_cast<const float*>(scales_v);
    const uint64_t rows = (WBITS == 4) ? K / 2 : K;
    TensorMap tm, tms, tmz;
    if (int e = get_tensor_map_2d_u8(ctx, B, rows, N, N, GV_ROWS, GV_BOX_COLS, true, &tm)) return e;
    tms = tm;                                     // W8 has no scale tiles; the kernel never uses the map
    tmz = tm;
    // rows of A are independent: M > 16 is served in slabs of 16 rows
    const int kps_d = GV_ROWS * (WBITS == 4 ? 2 : 1);
    const int k_pad = ceil_div(K, kps_d) * kps_d;
    const size_t slab_bytes = static_cast<size_t>(k_pad) * 8 * gv_jb_for(GV_MAX_M);
    uint8_t* const dig = static_cast<uint8_t*>(ctx->scratch);
    float* const inv = reinterpret_cast<float*>(dig + GV_DIG_BYTES - GV_INV_BYTES);
    // A prologue is applied where the digits are made, by the digit pass; a slab of one or two rows
    // makes its own digits inside the GEMV kernel and has no such hook.
    if (prologue != GV_PRO_NONE && jb_for(M - ((M - 1) / GV_MAX_M) * GV_MAX_M) == 1) return LHB_ERR_UNSUPPORTED;
    // The digit array holds a few slabs at a time (all of them unless K is very long).
    if (ctx->scratch_bytes < GV_DIG_BYTES || (M > 2 && slab_bytes > GV_DIG_BYTES - GV_INV_BYTES)) return LHB_ERR_SCRATCH;
    const int rows_per_pass =
        M > 2 ? std::min<int>(GV_INV_BYTES / 4, static_cast<int>((GV_DIG_BYTES - GV_INV_BYTES) / slab_bytes) * GV_MAX_M) : M;
    int pass0 = 0;                                  // first row of the current digit pass
    for (int m0 = 0; m0 < M; m0 += GV_MAX_M) {
        if (M > 2 && (m0 == 0 || m0 - pass0 >= rows_per_pass)) {
            // digits of the next rows, once, for all CTAs of the GEMV launches that follow
            pass0 = m0;
            const int rows = std::min(rows_per_pass, M - pass0);
            cudaLaunchConfig_t dc = {};
            dc.gridDim = dim3(rows, 1, 1);
            dc.blockDim = dim3(1024, 1, 1);
            dc.stream = st;
            cudaLaunchAttribute da[1];
            da[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            da[0].val.programmaticStreamSerializationAllowed = 1;
            dc.attrs = da;
            dc.numAttrs = 1;
            const int64_t row_len = (prologue == GV_PRO_SWIGLU) ? 2 * static_cast<int64_t>(K) : K;
            LHB_CUDA(cudaLaunchKernelEx(&dc, gemv_digits_kernel<WBITS>, A + pass0 * row_len, rows, K, k_pad,
                                        slab_bytes, dig, inv, prologue, gamma, eps));
        }
        const int m = std::min(GV_MAX_M, M - m0);
        const int jb = jb_for(m);
        GemvPlan pl = plan_gemv(WBITS, jb, N, K, WBITS == 4 ? G : 1, ctx->sm_count, ASYM);
        if (!pl.ok) return LHB_ERR_UNSUPPORTED;
        if (pl.col_tiles > static_cast<int>(ctx->counters_len)) return LHB_ERR_UNSUPPORTED;
        if (static_cast<size_t>(pl.col_tiles) * pl.max_contrib * m * GV_COLS * sizeof(float) >
            ctx->scratch_bytes - GV_DIG_BYTES)
            return LHB_ERR_SCRATCH;
        if (ASYM && m0 == 0) {
            if (int e = get_tensor_map_2d_f16(ctx, scales_v, K / G, N, static_cast<uint64_t>(N) * 2, 1, GV_COLS, &tms))
                return e;
            if (int e = get_tensor_map_2d_f16(ctx, zeros, K / G, N, static_cast<uint64_t>(N) * 2, 1, GV_COLS, &tmz))
                return e;
        } else if (WBITS == 4 && m0 == 0) {
            if (int e = get_tensor_map_2d_f32(ctx, scales, K / G, N, static_cast<uint64_t>(N) * 4, pl.srows,
                                              GV_COLS, &tms))
                return e;
            tmz = tms;
        }
        GemvParams p{};
        p.A = A + static_cast<int64_t>(m0) * K;
        p.scales = scales;
        p.C = C + static_cast<int64_t>(m0) * N;
        p.M = m; p.N = N; p.K = K; p.G = G; p.alpha = alpha; p.beta = beta;
        p.digits = dig + ((m0 - pass0) / GV_MAX_M) * slab_bytes;
        p.inv_scale = inv + (m0 - pass0);
        int e;
        if (ASYM) {
            if (jb == 1) e = launch_gemv_t<4, 1, true, ASYM>(ctx, tm, tms, tmz, p, pl, st);
            else if (jb == 2) e = launch_gemv_t<4, 2, true, ASYM>(ctx, tm, tms, tmz, p, pl, st);
            else if (jb == 3) e = launch_gemv_t<4, 3, true, ASYM>(ctx, tm, tms, tmz, p, pl, st);
            else e = launch_gemv_t<4, 6, true, ASYM>(ctx, tm, tms, tmz, p, pl, st);
        } else if (WBITS == 4 && G >= 128) {
            if (jb == 1) e = launch_gemv_t<WBITS, 1, WBITS == 4>(ctx, tm, tms, tmz, p, pl, st);
            else if (jb == 2) e = launch_gemv_t<WBITS, 2, WBITS == 4>(ctx, tm, tms, tmz, p, pl, st);
            else if (jb == 3) e = launch_gemv_t<WBITS, 3, WBITS == 4>(ctx, tm, tms, tmz, p, pl, st);
            else e = launch_gemv_t<WBITS, 6, WBITS == 4>(ctx, tm, tms, tmz, p, pl, st);
        } else {
            if (jb == 1) e = launch_gemv_t<WBITS, 1, false>(ctx, tm, tms, tmz, p, pl, st);
            else if (jb == 2) e = launch_gemv_t<WBITS, 2, false>(ctx, tm, tms, tmz, p, pl, st);
            else if (jb == 3) e = launch_gemv_t<WBITS, 3, false>(ctx, tm, tms, tmz, p, pl, st);
            else e = launch_gemv_t<WBITS, 6, false>(ctx, tm, tms, tmz, p, pl, st);
        }
        if (e) return e;
    }
    return LHB_OK;
}

int launch_w4a16_fast(lhb_ctx* ctx, const float* A, const uint8_t* Bp, const float* Bs, float* C,
                      int M, int N, int K, int G, float alpha, float beta, cudaStream_t st) {
    return launch_gemv<4>(ctx, A, Bp, Bs, nullptr, C, M, N, K, G, alpha, beta, st);
}

// asymmetric int4: the decode kernel serves group_size 128 (one group per 128-k stage)
bool w4a16_asym_fast_ok(int M, int N, int K, int G) {
    if (M < 1 || M > 1024 || (N % 16) != 0 || (K % 128) != 0 || G != 128) return false;
    if (M > 2 && static_cast<size_t>(K) * 48 > GV_DIG_BYTES - GV_INV_BYTES) return false;
    return plan_gemv(4, jb_for(std::min(M, GV_MAX_M)), N, K, G, 148, true).ok;
}
int launch_w4a16_asym_fast(lhb_ctx* ctx, const float* A, const uint8_t* Bp, const uint16_t* Bs, const uint16_t* Bz,
                           float* C, int M, int N, int K, int G, float alpha, float beta, cudaStream_t st) {
    return launch_gemv<4, true>(ctx, A, Bp, Bs, Bz, C, M, N, K, G, alpha, beta, st);
}

// gemm_w4a16_groupwise with RMSNorm or SwiGLU applied to the activations on the way in
int launch_w4a16_fast_prologue(lhb_ctx* ctx, const float* X, int prologue, const float* gamma, float eps,
                               const uint8_t* Bp, const float* Bs, float* C, int M, int N, int K, int G, float alpha,
                               float beta, cudaStream_t st) {
    return launch_gemv<4>(ctx, X, Bp, Bs, nullptr, C, M, N, K, G, alpha, beta, st, prologue, gamma, eps);
}

int launch_w8a16_fast(lhb_ctx* ctx, const float* A, const int8_t* Bq, const float* Bs, float* C,
                      int M, int N, int K, float alpha, float beta, cudaStream_t st) {
    return launch_gemv<8>(ctx, A, Bq, Bs, nullptr, C, M, N, K, 0, alpha, beta, st);
}

}  // namespace lhb

#ifdef LHB_GEMV_TRACE
extern "C" __attribute__((visibility("default"))) int lhb_debug_gemv_trace(void* host_out) {
    return static_cast<int>(cudaMemcpyFromSymbol(host_out, lhb::g_gv_trace, sizeof(lhb::g_gv_trace)));
}
#endif

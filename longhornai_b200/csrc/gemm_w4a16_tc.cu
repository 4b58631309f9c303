// W4A16 group-wise GEMM for a few dozen activation rows (decode batches, small prefill
// chunks) on the 5th-generation tensor cores.
//
// Semantics are the reference's gemm_w4a16_groupwise (src/kernels/gemm_quant.cpp:119-173;
// packing src/kernels/quantization.cpp:66-107): C = alpha * A * dequant(B) + beta * C with
// A fp32 [M, K], B packed int4 [K/2, N] (low nibble = even k, two's complement) and fp32
// scales [K/G, N].  The reference multiplies fp32 activations by fp32 dequantised weights;
// tensor cores have no fp32 operands, so the product is rebuilt exactly from integers:
//
//   * every activation row is scaled by a power of two so that its maximum lies in
//     [2^21, 2^22), rounded to an integer and split into three signed 8-bit digits
//     (iv = 65536*d2 + 256*d1 + d0; w4tc_digits_kernel, which also applies an optional
//     RMSNorm / SwiGLU to the row first);
//   * converter warps expand each 128-k x 128-column tile of nibbles into int8 (16 * q: a
//     shift and a mask per four weights) in shared memory;
//   * kind::i8 MMAs accumulate digit x weight products in int32 in TMEM, exactly.  The MMA
//     shape is [128 weight columns] x [3 digits * rows] x [32 k], the weights on the
//     128-lane side so that the per-column group scale is a per-thread constant of the
//     epilogue;
//   * after every group of 128 k the epilogue folds
//         acc[m] += (scale[g][n] / 16) * (65536*S2 + 256*S1 + S0)
//     in fp32 registers (the int32 sums are below 2^22 and convert exactly) and, at the end of
//     its K range, multiplies by the row's inverse power of two.
//
// The only roundings are the 22-bit activation grid (2^-22 of the row maximum), the fold
// (three fp32 FMAs per group) and the final scale - fewer than the reference's K sequential
// fp32 additions.  HBM traffic is the packed weights, read once.
//
// Work is split as in the GEMV kernel: a unit is 128 k x 256 columns (16 KiB of nibbles, two
// 128-column MMA tiles that share one digit tile); the units, ordered column tile by column
// tile, are dealt out to one CTA per SM; a CTA that holds only part of a column tile's K
// leaves its partial sums in scratch (same counters and scratch region as the GEMV kernel).
// When the grid is a whole number of CTAs per column tile - the usual case: the host picks
// such a grid whenever it keeps three quarters of the SMs busy - the contributors of a tile
// wait (bounded) until all of their partials are in memory and each adds up its share of the
// [M][256] outputs, in contributor order; all of them are resident, the grid being at most
// one CTA per SM.  Otherwise the last CTA to arrive at a tile adds everything up alone.
// Either way the order of the additions is fixed, so results do not vary from run to run.
//
// Warp roles (512 threads): 0 weight TMA producer, 1 MMA issuer, 2 TMEM allocator, 3 digit-tile
// TMA producer, 4-7 and 8-11 epilogue of the first / second 128-column half (TMEM lane quarter =
// warp % 4), 12-15 nibble -> int8 converters.
// Every wait is bounded (ptx::mbar_wait): a timeout sets the context's status word, the roles
// fall through to the common exit and TMEM is freed.
#include <algorithm>
#include <cstdlib>

#include "common.cuh"
#include "dispatch.h"
#include "ptx.cuh"

namespace lhb {

constexpr int TC_COLS = 256;                 // columns per unit
constexpr int TC_ROWS = 64;                  // byte-rows per unit (128 k)
constexpr int TC_RAW_BYTES = TC_COLS * TC_ROWS;          // 16 KiB
constexpr int TC_A_BYTES = 128 * 128;                    // one 128-k x 128-column int8 operand: 16 KiB
constexpr int TC_A_SLOTS = 4;                            // two units: one being multiplied, one being converted
constexpr int TC_B_STAGES = 5;
constexpr int TC_THREADS = 512;
constexpr int TC_CONV_WARPS = 4;
constexpr size_t TC_DIG_BYTES = (size_t(4) << 20) - 4096;   // digit region at the head of the scratch arena
constexpr size_t TC_SCRATCH_HEAD = size_t(4) << 20;         // its last 4 KiB: one fp32 factor per row of a pass

__host__ __device__ constexpr int tc_b_bytes(int mp) { return 3 * mp * 128; }         // [3*mp rows][128 k] int8
__host__ __device__ constexpr int tc_raw_stages(int mp) { return mp <= 16 ? 7 : 5; }
constexpr int TC_SC_DEPTH = 8;                           // group-scale ring: units ahead of the epilogue
__host__ __device__ constexpr size_t tc_smem(int mp) {
    return 1024 + size_t(TC_A_SLOTS) * TC_A_BYTES + size_t(TC_B_STAGES) * tc_b_bytes(mp) +
           size_t(tc_raw_stages(mp)) * TC_RAW_BYTES + size_t(TC_SC_DEPTH) * TC_COLS * 4 + 512;
}

enum { TC_PRO_NONE = 0, TC_PRO_RMSNORM = 1, TC_PRO_SWIGLU = 2 };

// Development builds (-DLHB_W4TC_TRACE): %globaltimer stamps per CTA, role and unit.
#ifdef LHB_W4TC_TRACE
__device__ unsigned long long g_tc_trace[160][4][64];
#define TC_STAMP(role, idx)                                                                  \
    do {                                                                                     \
        if (blockIdx.x < 160 && (idx) < 64) g_tc_trace[blockIdx.x][role][idx] = ptx::global_timer_ns(); \
    } while (0)
#else
#define TC_STAMP(role, idx) do { } while (0)
#endif

// ---- activation digits ------------------------------------------------------------------
// One CTA per row.  Output: int8 [slab][3*MP][K], row d*MP + m of a slab = digit d (0 = lowest)
// of its row m; inv_scale[row] = the inverse of the row's power-of-two factor.
// Rows of up to 16384 elements stay in registers between the passes.
__global__ void __launch_bounds__(1024)
w4tc_digits_kernel(const float* __restrict__ A, int K, int mp, int8_t* __restrict__ digits,
                   float* __restrict__ inv_scale, int prologue, const float* __restrict__ gamma, float eps) {
    __shared__ unsigned s_max[32];
    __shared__ float s_sum[32];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");      // A comes from the kernel before; so may readers of `digits`
    const int row_g = blockIdx.x, slab = row_g / mp, m = row_g - slab * mp;
    int8_t* d0_row = digits + (static_cast<int64_t>(slab) * 3 * mp + m) * K;
    const int64_t plane = static_cast<int64_t>(mp) * K;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t row_len = (prologue == TC_PRO_SWIGLU) ? 2 * static_cast<int64_t>(K) : K;
    const float* row = A + static_cast<int64_t>(row_g) * row_len;
    constexpr int DC = 4;
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
    if (prologue == TC_PRO_RMSNORM) {
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
    auto transform = [&](float4 v, int k) {
        if (prologue == TC_PRO_RMSNORM) {
            const float4 g = *reinterpret_cast<const float4*>(gamma + k);
            v.x = __fmul_rn(__fmul_rn(v.x, inv_rms), g.x); v.y = __fmul_rn(__fmul_rn(v.y, inv_rms), g.y);
            v.z = __fmul_rn(__fmul_rn(v.z, inv_rms), g.z); v.w = __fmul_rn(__fmul_rn(v.w, inv_rms), g.w);
        } else if (prologue == TC_PRO_SWIGLU) {
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
            if (k < K && prologue != TC_PRO_NONE) hv[i] = transform(hv[i], k);
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
    auto put = [&](int k, float4 v) {
        // iv = rint(v * scl) = 65536*d2 + 256*d1 + d0 with d0, d1 in [-128, 127] and |d2| <= 64: the low
        // byte of an integer, read as signed, is its balanced digit, and what remains is divisible by 256
        const int iv[4] = {__float2int_rn(v.x * scl), __float2int_rn(v.y * scl), __float2int_rn(v.z * scl),
                           __float2int_rn(v.w * scl)};
        uint32_t w0 = 0, w1 = 0, w2 = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int lo = static_cast<int>(static_cast<int8_t>(iv[j]));
            const int iv2 = (iv[j] - lo) >> 8;
            const int mid = static_cast<int>(static_cast<int8_t>(iv2));
            const int hi = (iv2 - mid) >> 8;
            w0 |= (static_cast<uint32_t>(lo) & 0xffu) << (8 * j);
            w1 |= (static_cast<uint32_t>(mid) & 0xffu) << (8 * j);
            w2 |= (static_cast<uint32_t>(hi) & 0xffu) << (8 * j);
        }
        *reinterpret_cast<uint32_t*>(d0_row + k) = w0;
        *reinterpret_cast<uint32_t*>(d0_row + plane + k) = w1;
        *reinterpret_cast<uint32_t*>(d0_row + 2 * plane + k) = w2;
    };
    if (cached) {
#pragma unroll
        for (int i = 0; i < DC; ++i) {
            const int k = threadIdx.x * 4 + i * 4096;
            if (k < K) put(k, hv[i]);
        }
    } else {
        for (int k = threadIdx.x * 4; k < K; k += 4096) put(k, transform(*reinterpret_cast<const float4*>(row + k), k));
    }
}

// ---- the GEMM ---------------------------------------------------------------------------

struct W4TcParams {
    const float* scales;     // [K/G, N]
    float* C;                // [M, N], this slab's first row
    int M, N, K, G;          // M = rows of this slab (<= MP)
    float alpha, beta;
    int S;                   // units per column tile = K / 128
    int units;               // column tiles * S
    int max_contrib;         // partial slots per column tile in scratch
    float* partial;          // scratch [column tile][max_contrib][M][256]
    int* counters;           // one per column tile, zero between calls
    int coop_sum;            // every CTA's units lie in one column tile (a whole number of CTAs per tile): the
                             // contributors of a tile wait for each other and each adds up its share of the outputs
    int* status;
    const float* inv_scale;  // [M]
    int dig_row0;            // first row of this slab in the digit tensor
    // Sharded use (peer_world > 0): the final values also go to columns [peer_col0, peer_col0 + N) of every
    // rank's row-major [rows, peer_ld] matrix (peer_dst[w], this slab's first row added by the kernel), and
    // the CTA that completes a column tile then adds one to counter `peer_rank` of every rank (peer_flags[w]).
    float* const* peer_dst;
    uint32_t* const* peer_flags;
    int peer_world, peer_rank, peer_ld, peer_col0, peer_row0;
};

// PEER is a template parameter of the kernel: the unsharded instantiation carries none of this code
#define TC_PW(p) (PEER ? (p).peer_world : 0)

// one arrival at every rank of a sharded GEMM, by the thread that has fenced the CTA's stores
__device__ __forceinline__ void tc_peer_signal(const W4TcParams& p) {
    __threadfence_system();
    for (int w = 0; w < p.peer_world; ++w)
        asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(p.peer_flags[w] + p.peer_rank) : "memory");
}

// int8 x int8 -> int32 (bits 4-5 = 2; formats at bits 7-9 and 10-12 = 1), A = weights MN-major
// (bit 15), B = digits K-major, N >> 3 at bit 17, M = 128 >> 4 at bit 24
__host__ __device__ constexpr uint32_t tc_idesc(int n) {
    return (2u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (static_cast<uint32_t>(n >> 3) << 17) |
           (static_cast<uint32_t>(128 >> 4) << 24);
}

// exact int32 -> fp32 for |v| < 2^22 without the conversion pipe
__device__ __forceinline__ float tc_int_to_float(uint32_t v) {
    return __uint_as_float(v + 0x4B400000u) - 12582912.0f;
}

// The last contributor to a column tile adds the partial sums up and writes C.  NT threads share the
// [M][256] outputs as float4s, whatever columns they held before: each takes up to four of them at a
// time and adds the contributors' float4s in contributor order, Y contributors' loads in flight per
// round trip to L2.  A CTA's last segment is summed by all of its 512 threads after the role loops
// (the other roles have nothing left to do), five contributors per round trip: with nine CTAs per
// column tile the sum costs two round trips instead of six, which is what the end of a short GEMM
// (the o and QKV projections of a decode step: 3-5 units per CTA) spends its time on.
template <bool PEER, int NT, int Y>
__device__ __forceinline__ void tc_sum_partials(const W4TcParams& p, const float* tile_slots, int tile_col0,
                                                int n_contrib, int et) {
    const int n_out = p.M * (TC_COLS / 4);
    for (int e0 = et; e0 < n_out; e0 += 4 * NT) {
        float4 sum[4];
#pragma unroll
        for (int x = 0; x < 4; ++x) sum[x] = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j < n_contrib; j += Y) {
            float4 v[Y][4];
#pragma unroll
            for (int y = 0; y < Y; ++y) {
                const float* slot = tile_slots + static_cast<int64_t>(min(j + y, n_contrib - 1)) * p.M * TC_COLS;
#pragma unroll
                for (int x = 0; x < 4; ++x)       // clamped, unconditional: the loads overlap
                    v[y][x] = __ldcg(reinterpret_cast<const float4*>(slot) + min(e0 + NT * x, n_out - 1));
            }
#pragma unroll
            for (int y = 0; y < Y; ++y) {
                if (j + y < n_contrib) {
#pragma unroll
                    for (int x = 0; x < 4; ++x) {
                        sum[x].x += v[y][x].x; sum[x].y += v[y][x].y; sum[x].z += v[y][x].z; sum[x].w += v[y][x].w;
                    }
                }
            }
        }
        float4 old[4];
        if (p.beta != 0.0f) {
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                const int e = min(e0 + NT * x, n_out - 1), m = e >> 6, c = (e & 63) * 4;
                old[x] = (tile_col0 + c < p.N) ? *reinterpret_cast<const float4*>(p.C + m * p.N + tile_col0 + c)
                                               : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            const int e = e0 + NT * x, m = e >> 6, c = (e & 63) * 4;
            if (e < n_out && tile_col0 + c < p.N) {       // N % 16 == 0: whole float4 in range
                float4 r;
                if (p.beta == 0.0f) {
                    r = make_float4(p.alpha * sum[x].x, p.alpha * sum[x].y, p.alpha * sum[x].z, p.alpha * sum[x].w);
                } else {
                    r.x = fmaf(p.beta, old[x].x, p.alpha * sum[x].x); r.y = fmaf(p.beta, old[x].y, p.alpha * sum[x].y);
                    r.z = fmaf(p.beta, old[x].z, p.alpha * sum[x].z); r.w = fmaf(p.beta, old[x].w, p.alpha * sum[x].w);
                }
                *reinterpret_cast<float4*>(p.C + m * p.N + tile_col0 + c) = r;
                for (int w = 0; w < TC_PW(p); ++w)
                    *reinterpret_cast<float4*>(p.peer_dst[w] + static_cast<int64_t>(p.peer_row0 + m) * p.peer_ld +
                                               p.peer_col0 + tile_col0 + c) = r;
            }
        }
    }
}

// The shared form of that sum: contributor `ci` of `n_contrib` adds up outputs [ci, ci + 1) * n_out / n_contrib
// of the tile once every contributor's partial is in memory - a few kilobytes per CTA instead of
// n_contrib * 32 KiB into one SM, which is a bandwidth limit of that SM (2.4 us for nine contributors),
// not a latency.  Same order of additions as tc_sum_partials.
template <bool PEER>
__device__ __forceinline__ void tc_sum_slice(const W4TcParams& p, const float* tile_slots, int tile_col0, int n_contrib,
                                             int ci, int tid) {
    const int n_out = p.M * (TC_COLS / 4);
    const int lo = static_cast<int>(static_cast<int64_t>(ci) * n_out / n_contrib);
    const int hi = static_cast<int>(static_cast<int64_t>(ci + 1) * n_out / n_contrib);
    for (int e = lo + tid; e < hi; e += TC_THREADS) {
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j < n_contrib; j += 8) {
            float4 v[8];
#pragma unroll
            for (int y = 0; y < 8; ++y)
                v[y] = __ldcg(reinterpret_cast<const float4*>(tile_slots + static_cast<int64_t>(min(j + y, n_contrib - 1)) * p.M * TC_COLS) + e);
#pragma unroll
            for (int y = 0; y < 8; ++y)
                if (j + y < n_contrib) { sum.x += v[y].x; sum.y += v[y].y; sum.z += v[y].z; sum.w += v[y].w; }
        }
        const int m = e >> 6, c = (e & 63) * 4;
        if (tile_col0 + c >= p.N) continue;               // N % 16 == 0: whole float4 in range
        float4 r;
        if (p.beta == 0.0f) {
            r = make_float4(p.alpha * sum.x, p.alpha * sum.y, p.alpha * sum.z, p.alpha * sum.w);
        } else {
            const float4 old = *reinterpret_cast<const float4*>(p.C + m * p.N + tile_col0 + c);
            r.x = fmaf(p.beta, old.x, p.alpha * sum.x); r.y = fmaf(p.beta, old.y, p.alpha * sum.y);
            r.z = fmaf(p.beta, old.z, p.alpha * sum.z); r.w = fmaf(p.beta, old.w, p.alpha * sum.w);
        }
        *reinterpret_cast<float4*>(p.C + m * p.N + tile_col0 + c) = r;
        for (int w = 0; w < TC_PW(p); ++w)
            *reinterpret_cast<float4*>(p.peer_dst[w] + static_cast<int64_t>(p.peer_row0 + m) * p.peer_ld + p.peer_col0 +
                                       tile_col0 + c) = r;
    }
}

__device__ __forceinline__ void tc_epi_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

template <int MP, bool PEER>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_w4a16_tc_kernel(const __grid_constant__ TensorMap tmW, const __grid_constant__ TensorMap tmD,
                     const W4TcParams p) {
    constexpr int NMMA = 3 * MP;                       // MMA N: three digit rows per activation row
    constexpr int RS = tc_raw_stages(MP);
    constexpr int BS = TC_B_STAGES;
    constexpr int B_BYTES = tc_b_bytes(MP);
    constexpr int TSTRIDE = MP <= 16 ? 64 : 128;       // columns between accumulators
    constexpr int TCOLS = 4 * TSTRIDE;                 // four accumulators of NMMA columns (two units in flight)
    extern __shared__ uint8_t tc_smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* a_ring = smem;
    uint8_t* b_ring = a_ring + TC_A_SLOTS * TC_A_BYTES;
    uint8_t* raw_ring = b_ring + BS * B_BYTES;
    float* sc_ring = reinterpret_cast<float*>(raw_ring + RS * TC_RAW_BYTES);       // [TC_SC_DEPTH][256]
    uint64_t* bars = reinterpret_cast<uint64_t*>(sc_ring + TC_SC_DEPTH * TC_COLS);
    // barriers: raw_full[RS] raw_empty[RS] a_full[3] a_empty[3] b_full[BS] b_empty[BS] t_full[4] t_empty[4]
    constexpr int NBARS = 2 * RS + 2 * TC_A_SLOTS + 2 * BS + 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NBARS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* epi_flag = const_cast<int*>(reinterpret_cast<volatile int*>(tmem_slot + 2));
    int* final_tile = const_cast<int*>(reinterpret_cast<volatile int*>(tmem_slot + 3));   // column tile this CTA sums at its end, or -1
    float* inv_s = reinterpret_cast<float*>(tmem_slot + 4);          // [MP]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar0 = ptx::smem_u32(bars);
    auto raw_full = [&](int s) { return bar0 + 8 * s; };
    auto raw_empty = [&](int s) { return bar0 + 8 * (RS + s); };
    auto a_full = [&](int s) { return bar0 + 8 * (2 * RS + s); };
    auto a_empty = [&](int s) { return bar0 + 8 * (2 * RS + TC_A_SLOTS + s); };
    auto b_full = [&](int s) { return bar0 + 8 * (2 * RS + 2 * TC_A_SLOTS + s); };
    auto b_empty = [&](int s) { return bar0 + 8 * (2 * RS + 2 * TC_A_SLOTS + BS + s); };
    auto t_full = [&](int s) { return bar0 + 8 * (2 * RS + 2 * TC_A_SLOTS + 2 * BS + s); };
    auto t_empty = [&](int s) { return bar0 + 8 * (2 * RS + 2 * TC_A_SLOTS + 2 * BS + 4 + s); };

    // this CTA's units [u0, u1), ordered column tile by column tile
    const int S = p.S;
    const int u0 = static_cast<int>(static_cast<int64_t>(blockIdx.x) * p.units / gridDim.x);
    const int u1 = static_cast<int>(static_cast<int64_t>(blockIdx.x + 1) * p.units / gridDim.x);
    const int n_units = u1 - u0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < RS; ++s) { ptx::mbar_init(raw_full(s), 1); ptx::mbar_init(raw_empty(s), TC_CONV_WARPS); }
        for (int s = 0; s < TC_A_SLOTS; ++s) { ptx::mbar_init(a_full(s), TC_CONV_WARPS); ptx::mbar_init(a_empty(s), 1); }
        for (int s = 0; s < BS; ++s) { ptx::mbar_init(b_full(s), 1); ptx::mbar_init(b_empty(s), 1); }
        for (int s = 0; s < 4; ++s) { ptx::mbar_init(t_full(s), 1); ptx::mbar_init(t_empty(s), 128); }
        *abort_flag = 0;
        *epi_flag = 0;
        *final_tile = -1;
        ptx::fence_mbar_init();
        ptx::prefetch_tmap(&tmW);
        ptx::prefetch_tmap(&tmD);
        // The weights depend on nothing an earlier kernel of the stream writes: the first ring-full is
        // requested before the programmatic dependency below resolves.
        const int first = min(n_units, RS);
        for (int i = 0; i < first; ++i) {
            const int u = u0 + i, tile = u / S, g = u - tile * S;
            ptx::mbar_expect_tx(raw_full(i), TC_RAW_BYTES);
            ptx::tma_load_2d(ptx::smem_u32(raw_ring + i * TC_RAW_BYTES), &tmW, tile * TC_COLS, g * TC_ROWS, raw_full(i));
        }
    }
    if (warp == 2) {
        ptx::tmem_alloc(ptx::smem_u32(tmem_slot), TCOLS);
        ptx::tmem_relinquish();
    }
    if (threadIdx.x == 0) TC_STAMP(3, 0);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Digits, C, scratch, counters and the row factors belong to earlier kernels of the stream: every role
    // that touches them waits for the programmatic dependency here.  The weight producer and the converters
    // touch only the weights and shared memory, so the first two units are converted while the previous
    // kernel drains.
    if (warp != 0 && warp < 12) asm volatile("griddepcontrol.wait;" ::: "memory");
    if (threadIdx.x == 32) TC_STAMP(3, 1);

    if (warp == 0) {
        // ---- weight producer: refill ring slots as the converters release them ----
        if (lane == 0) {
            int issued = min(n_units, RS);
            for (int i = RS; i < n_units; ++i) {
                const int s = i % RS;
                if (!ptx::mbar_wait(raw_empty(s), ((i / RS) & 1) ^ 1, abort_flag, p.status)) break;
                const int u = u0 + i, tile = u / S, g = u - tile * S;
                ptx::mbar_expect_tx(raw_full(s), TC_RAW_BYTES);
                ptx::tma_load_2d(ptx::smem_u32(raw_ring + s * TC_RAW_BYTES), &tmW, tile * TC_COLS, g * TC_ROWS, raw_full(s));
                issued = i + 1;
            }
            if (*abort_flag) {
                // a wait ran out: let the copies still in flight land before the CTA exits
                for (int i = max(0, issued - RS); i < issued; ++i) {
                    const uint64_t t0 = ptx::global_timer_ns();
                    while (!ptx::mbar_try_wait(raw_full(i % RS), (i / RS) & 1))
                        if (ptx::global_timer_ns() - t0 > 200000000ull) break;
                }
            }
        }
    } else if (warp == 3) {
        // ---- digit-tile producer: [3*MP rows][128 k] int8 per unit ----
        if (lane == 0) {
            int issued = 0;
            for (int i = 0; i < n_units; ++i) {
                const int s = i % BS;
                if (!ptx::mbar_wait(b_empty(s), ((i / BS) & 1) ^ 1, abort_flag, p.status)) break;
                const int u = u0 + i, tile = u / S, g = u - tile * S;
                const uint32_t dst = ptx::smem_u32(b_ring + s * B_BYTES);
                ptx::mbar_expect_tx(b_full(s), B_BYTES);
                ptx::tma_load_2d(dst, &tmD, g * 128, p.dig_row0, b_full(s));
                issued = i + 1;
            }
            if (*abort_flag) {
                for (int i = max(0, issued - BS); i < issued; ++i) {
                    const uint64_t t0 = ptx::global_timer_ns();
                    while (!ptx::mbar_try_wait(b_full(i % BS), (i / BS) & 1))
                        if (ptx::global_timer_ns() - t0 > 200000000ull) break;
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer: per unit, two 128-column tiles x eight k16 steps ----
        if (lane == 0) {
            for (int i = 0; i < n_units; ++i) {
                const int bs = i % BS;
                if (!ptx::mbar_wait(b_full(bs), (i / BS) & 1, abort_flag, p.status)) break;
                if (i < 14) TC_STAMP(3, 8 + 4 * i);
                const uint32_t sb = ptx::smem_u32(b_ring + bs * B_BYTES);
                bool ok = true;
#pragma unroll 1
                for (int sub = 0; sub < 2; ++sub) {
                    const int n = 2 * i + sub, as = n % TC_A_SLOTS, tb = n & 3;
                    if (!ptx::mbar_wait(a_full(as), (n / TC_A_SLOTS) & 1, abort_flag, p.status)) { ok = false; break; }
                    if (i < 14) TC_STAMP(3, 8 + 4 * i + 1 + sub);
                    if (!ptx::mbar_wait(t_empty(tb), ((n >> 2) & 1) ^ 1, abort_flag, p.status)) { ok = false; break; }
                    if (i < 14 && sub == 1) TC_STAMP(3, 8 + 4 * i + 3);
                    ptx::tc_fence_after();
                    const uint32_t sa = ptx::smem_u32(a_ring + as * TC_A_BYTES);
                    const uint32_t d_tmem = tmem_base + tb * TSTRIDE;
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        // A: MN-major, one 128-column atom wide, 8-k atoms 1 KiB apart, 32 k per step
                        const uint64_t da = ptx::smem_desc_sw128(sa + kk * 4096, 16, 1024);
                        // B: K-major rows of 128 B (128 k), 8-row atoms 1 KiB apart; 32 B per step
                        const uint64_t db = ptx::smem_desc_sw128(sb + kk * 32, 16, 1024);
                        ptx::mma_i8_ss(d_tmem, da, db, tc_idesc(NMMA), kk != 0 ? 1u : 0u);
                    }
                    ptx::tc_commit(a_empty(as));
                    ptx::tc_commit(t_full(tb));
                }
                if (!ok) break;
                ptx::tc_commit(b_empty(bs));
                TC_STAMP(1, i);
            }
        }
    } else if (warp >= 12) {
        // ---- converters: nibbles of one unit -> two int8 operand tiles ----
        const int ct = threadIdx.x - 384;                    // 0..127
        for (int i = 0; i < n_units; ++i) {
            const int rs = i % RS;
            if (!ptx::mbar_wait(raw_full(rs), (i / RS) & 1, abort_flag, p.status)) break;
            const uint8_t* raw = raw_ring + rs * TC_RAW_BYTES;
            // both halves of the unit at once: eight 16-byte loads per thread in flight, one fence
            const int as0 = (2 * i) % TC_A_SLOTS, par = (((2 * i) / TC_A_SLOTS) & 1) ^ 1;
            if (!ptx::mbar_wait(a_empty(as0), par, abort_flag, p.status)) break;
            if (!ptx::mbar_wait(a_empty(as0 + 1), par, abort_flag, p.status)) break;
            uint8_t* at = a_ring + as0 * TC_A_BYTES;         // the second half's tile follows the first
            uint4 w[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int task = ct + 128 * (j & 3);         // 64 byte-rows x 8 chunks of 16 columns, per half
                w[j] = *reinterpret_cast<const uint4*>(raw + (task >> 3) * TC_COLS + (j >> 2) * 128 + (task & 7) * 16);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int task = ct + 128 * (j & 3);
                const int r = task >> 3, ch = task & 7;
                // low nibbles = row k = 2r, high nibbles = row k + 1, both as 16 * q in int8
                const uint4 ev = make_uint4((w[j].x << 4) & 0xf0f0f0f0u, (w[j].y << 4) & 0xf0f0f0f0u,
                                            (w[j].z << 4) & 0xf0f0f0f0u, (w[j].w << 4) & 0xf0f0f0f0u);
                const uint4 od = make_uint4(w[j].x & 0xf0f0f0f0u, w[j].y & 0xf0f0f0f0u, w[j].z & 0xf0f0f0f0u,
                                            w[j].w & 0xf0f0f0f0u);
                // row k of the tile: 128 B, atom k / 8, 16-byte chunk swizzled with k % 8
                const int k = 2 * r, kin = k & 7;
                uint8_t* base = at + (j >> 2) * TC_A_BYTES + (k >> 3) * 1024;
                *reinterpret_cast<uint4*>(base + kin * 128 + ((ch ^ kin) << 4)) = ev;
                *reinterpret_cast<uint4*>(base + (kin + 1) * 128 + ((ch ^ (kin + 1)) << 4)) = od;
            }
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                ptx::mbar_arrive(a_full(as0));
                ptx::mbar_arrive(a_full(as0 + 1));
                ptx::mbar_arrive(raw_empty(rs));
            }
            if (threadIdx.x == 384) TC_STAMP(0, i);
        }
    } else if (warp >= 4 && warp < 12) {
        // ---- epilogue: two sets of four warps, set `sub` owns the 128-column half `sub` of every unit; it
        // folds each unit's sums into fp32 registers and hands a segment over at its end ----
        const int sub = (warp - 4) >> 2, q = warp & 3;
        const int cl = 32 * q + lane;                        // TMEM lane = column of the 128-column half
        const int et = threadIdx.x - 128;                    // 0..255
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(32 * q) << 16);
        if (et < MP) inv_s[et] = et < p.M ? p.inv_scale[et] : 0.0f;
        tc_epi_sync();
        float acc[MP];
        int i = 0, u = u0;
        bool alive = true;
        while (u < u1 && alive) {
            const int tile = u / S, s_begin = u - tile * S, s_end = min(S, s_begin + (u1 - u));
            const int col0 = tile * TC_COLS + sub * 128;     // first column of this set's half
            const bool valid = col0 + cl < p.N;
#pragma unroll
            for (int m = 0; m < MP; ++m) acc[m] = 0.0f;
            // Group scales: one per column and group, read from memory once per GEMM (always a DRAM
            // miss).  Every thread copies its own column's scale of the unit TC_SC_DEPTH - 1 ahead into
            // a shared-memory ring with cp.async and later reads back only what it wrote itself, so
            // the ring needs no barrier.
            float* my_sc = sc_ring + sub * 128 + cl;
            auto fetch_scale = [&](int g) {                  // one commit group per unit, even when nothing is copied
                if (valid && g < s_end) {
                    const float* sp = p.scales + static_cast<int64_t>((g * 128) / p.G) * p.N + col0 + cl;
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(ptx::smem_u32(my_sc + (g % TC_SC_DEPTH) * TC_COLS)),
                                 "l"(sp) : "memory");
                }
                asm volatile("cp.async.commit_group;" ::: "memory");
            };
            for (int j = 0; j < TC_SC_DEPTH - 1; ++j) fetch_scale(s_begin + j);
            const int n_slices = (p.M + 7) >> 3;             // 8 rows per slice
            for (int g = s_begin; g < s_end; ++g, ++i) {
                fetch_scale(g + TC_SC_DEPTH - 1);
                asm volatile("cp.async.wait_group %0;" ::"n"(TC_SC_DEPTH - 1) : "memory");
                const float sc = valid ? 0.0625f * my_sc[(g % TC_SC_DEPTH) * TC_COLS] : 0.0f;   // nibbles are carried as 16 * q
                const int n = 2 * i + sub, tb = n & 3;
                if (!ptx::mbar_wait(t_full(tb), (n >> 2) & 1, abort_flag, p.status)) { alive = false; break; }
                ptx::tc_fence_after();
                // rows 8c..8c+7 = one 8-column slice of each digit plane; the loads of slice c + 1 are in
                // flight while slice c is folded
                const uint32_t t0 = lane_base + tb * TSTRIDE;
                uint32_t r[2][3][8];
                ptx::tmem_ld_32x8(t0, r[0][0]);
                ptx::tmem_ld_32x8(t0 + MP, r[0][1]);
                ptx::tmem_ld_32x8(t0 + 2 * MP, r[0][2]);
#pragma unroll
                for (int c = 0; c < MP / 8; ++c) {
                    if (c < n_slices) {
                        ptx::tmem_ld_wait();
                        if (c + 1 < n_slices) {
                            if (c + 1 < MP / 8) {
                                ptx::tmem_ld_32x8(t0 + 8 * (c + 1), r[(c + 1) & 1][0]);
                                ptx::tmem_ld_32x8(t0 + MP + 8 * (c + 1), r[(c + 1) & 1][1]);
                                ptx::tmem_ld_32x8(t0 + 2 * MP + 8 * (c + 1), r[(c + 1) & 1][2]);
                            }
                        } else {                             // last slice read: the accumulator may be overwritten
                            ptx::tc_fence_before();
                            ptx::mbar_arrive(t_empty(tb));
                        }
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const float t = fmaf(65536.0f, tc_int_to_float(r[c & 1][2][e]),
                                                 fmaf(256.0f, tc_int_to_float(r[c & 1][1][e]),
                                                      tc_int_to_float(r[c & 1][0][e])));
                            acc[8 * c + e] = fmaf(sc, t, acc[8 * c + e]);
                        }
                    }
                }
                if (et == 0) TC_STAMP(2, i);
            }
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            if (et == 0) TC_STAMP(3, 2);
            if (!alive) break;

            // ---- end of this CTA's share of the column tile ----
            const bool whole = (s_begin == 0 && s_end == S);
            int cf = 0, n_contrib = 1;
            if (!whole) {                                    // contributors are the CTAs cf..cf + n_contrib - 1
                const int64_t P = gridDim.x;
                cf = static_cast<int>(((static_cast<int64_t>(tile) * S + 1) * P - 1) / p.units);
                const int cz = static_cast<int>(((static_cast<int64_t>(tile + 1) * S) * P - 1) / p.units);
                n_contrib = cz - cf + 1;
            }
            // partial slots hold [M][256] in column order; this thread's entries are column sub * 128 + cl
            float* slot_base = p.partial + (static_cast<int64_t>(tile) * p.max_contrib) * p.M * TC_COLS + sub * 128 + cl;
            float* my_slot = slot_base + static_cast<int64_t>(blockIdx.x - cf) * p.M * TC_COLS;
            // C[m][this lane's column] = alpha * val[m] + beta * C for the slab's rows.  The reads of C are
            // issued eight at a time without row guards (row index clamped), so that they overlap.
            auto store_rows = [&](const float (&val)[MP]) {
                float* cp = p.C + col0 + cl;
#pragma unroll
                for (int m0 = 0; m0 < MP; m0 += 8) {
                    if (m0 >= p.M) break;
                    float old[8];
                    if (p.beta != 0.0f) {
#pragma unroll
                        for (int m = 0; m < 8; ++m) old[m] = cp[min(m0 + m, p.M - 1) * p.N];     // slab rows * N < 2^31
                    }
#pragma unroll
                    for (int m = 0; m < 8; ++m) {
                        if (m0 + m < p.M) {
                            const float r = (p.beta == 0.0f) ? p.alpha * val[m0 + m] : fmaf(p.beta, old[m], p.alpha * val[m0 + m]);
                            cp[(m0 + m) * p.N] = r;
                            for (int w = 0; w < TC_PW(p); ++w)
                                p.peer_dst[w][static_cast<int64_t>(p.peer_row0 + m0 + m) * p.peer_ld + p.peer_col0 + col0 + cl] = r;
                        }
                    }
                }
            };
            if (valid) {
#pragma unroll
                for (int m = 0; m < MP; ++m) acc[m] *= inv_s[m];
                if (whole) {
                    store_rows(acc);
                } else {
#pragma unroll
                    for (int m = 0; m < MP; ++m)
                        if (m < p.M) my_slot[m * TC_COLS] = acc[m];
                }
            }
            if (whole && TC_PW(p) > 0) {                 // the tile is complete: tell every rank
                tc_epi_sync();
                if (et == 0) tc_peer_signal(p);
            }
            if (!whole && p.coop_sum) {
                // this CTA's only segment: count the arrival; the wait for the others and the sum follow the role loops
                tc_epi_sync();
                if (et == 0) {
                    __threadfence();
                    atomicAdd(p.counters + tile, 1);
                    *final_tile = tile;
                }
            } else if (!whole) {
                // the last contributor to arrive adds the partials up in contributor order and writes C;
                // one thread fences for the CTA on either side of the count
                const bool final_seg = (u + (s_end - s_begin) >= u1);   // nothing follows: the whole CTA sums, below
                tc_epi_sync();
                if (et == 0) {
                    __threadfence();
                    const int old = atomicAdd(p.counters + tile, 1);
                    const int last = (old == n_contrib - 1);
                    if (last) {
                        p.counters[tile] = 0;                // ready for the next call
                        __threadfence();
                    }
                    if (final_seg) {
                        *final_tile = last ? tile : -1;
                        *epi_flag = 0;
                    } else {
                        *epi_flag = last;
                    }
                }
                tc_epi_sync();
                if (*epi_flag) tc_sum_partials<PEER, 256, 3>(p, p.partial + (static_cast<int64_t>(tile) * p.max_contrib) * p.M * TC_COLS, tile * TC_COLS, n_contrib, et);
                tc_epi_sync();                               // epi_flag is free again
                if (TC_PW(p) > 0 && et == 0 && *epi_flag) tc_peer_signal(p);
            }
            if (et == 0) TC_STAMP(3, 3);
            u += s_end - s_begin;
        }
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 2) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, TCOLS);
    }
    // this CTA arrived last at the column tile its units ended in: all 512 threads add the partials up
    const int ft = *final_tile;
    if (ft >= 0 && !*abort_flag) {
        const int64_t P = gridDim.x;
        const int cf = static_cast<int>(((static_cast<int64_t>(ft) * S + 1) * P - 1) / p.units);
        const int cz = static_cast<int>(((static_cast<int64_t>(ft + 1) * S) * P - 1) / p.units);
        const int n_contrib = cz - cf + 1;
        const float* slots = p.partial + (static_cast<int64_t>(ft) * p.max_contrib) * p.M * TC_COLS;
        if (p.coop_sum) {
            // The counter counts arrivals (partials in memory) up to n_contrib and then departures; the
            // departures increment with wrap-around at 2 * n_contrib - 1, so the last one leaves zero behind
            // for the next call and nobody has to wait for the value it read (only the sharded form does:
            // the last to leave tells the other ranks).
            const unsigned wrap = 2u * static_cast<unsigned>(n_contrib) - 1u;
            if (threadIdx.x == 0) {
                const uint64_t t0 = ptx::global_timer_ns();
                while (ptx::ld_acquire_gpu(p.counters + ft) < n_contrib) {
                    if (ptx::global_timer_ns() - t0 > 1000000000ull) {      // a contributor never ran: report, do not hang
                        *abort_flag = 1;
                        atomicExch(p.status, static_cast<int>(LHB_ERR_TIMEOUT));
                        break;
                    }
                }
                TC_STAMP(3, 4);
            }
            __syncthreads();
            if (!*abort_flag) tc_sum_slice<PEER>(p, slots, ft * TC_COLS, n_contrib, static_cast<int>(blockIdx.x) - cf, threadIdx.x);
            if (TC_PW(p) > 0) {
                __syncthreads();
                if (threadIdx.x == 0) {
                    __threadfence_system();
                    const unsigned old = atomicInc(reinterpret_cast<unsigned*>(p.counters + ft), wrap);
                    if (old == wrap && !*abort_flag) tc_peer_signal(p);   // the last to leave: the tile is complete everywhere
                }
            } else if (threadIdx.x == 0) {
                // this thread's own outputs need no ordering against the count: the kernel's end publishes them
                asm volatile("red.relaxed.gpu.global.inc.u32 [%0], %1;" ::"l"(p.counters + ft), "r"(wrap) : "memory");
            }
        } else {
            tc_sum_partials<PEER, TC_THREADS, 5>(p, slots, ft * TC_COLS, n_contrib, threadIdx.x);
            if (TC_PW(p) > 0) {
                __syncthreads();
                if (threadIdx.x == 0) tc_peer_signal(p);
            }
        }
        if (threadIdx.x == 0) TC_STAMP(3, 3);
    }
}

// ---- host side --------------------------------------------------------------------------

static int tc_slab_rows(int M) { return M > 16 ? 32 : 16; }
static int tc_digit_rows(int mp) { return 3 * mp; }      // digit rows per slab

bool w4a16_tc_ok(int M, int N, int K, int G) {
    if (M < 1 || M > 65536 || N < 16 || (N % 16) != 0 || G < 128 || (G % 128) != 0 || K < G || (K % G) != 0) return false;
    // the digits of one slab must fit the head of the scratch arena
    return static_cast<size_t>(tc_digit_rows(tc_slab_rows(M))) * K <= TC_DIG_BYTES;
}

// programmatic dependent launch between the digit pass and the GEMMs; LHB_PDL=0 turns it off
static bool tc_pdl() { return knobs().pdl; }

int w4a16_tc_min_rows() { return knobs().w4tc_min_m; }

template <int MP, bool PEER>
static int launch_tc_slab(lhb_ctx* ctx, const TensorMap& tmW, const TensorMap& tmD, W4TcParams p, int ctas,
                          cudaStream_t st) {
    auto kern = gemm_w4a16_tc_kernel<MP, PEER>;
    static bool attr_set[64] = {};
    if (!attr_set[ctx->device & 63]) {
        LHB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(tc_smem(MP))));
        attr_set[ctx->device & 63] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas, 1, 1);
    cfg.blockDim = dim3(TC_THREADS, 1, 1);
    cfg.dynamicSmemBytes = tc_smem(MP);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tc_pdl() ? 1 : 0;
    LHB_CUDA(cudaLaunchKernelEx(&cfg, kern, tmW, tmD, p));
    return LHB_OK;
}

int launch_w4a16_tc(lhb_ctx* ctx, const float* A, const uint8_t* Bp, const float* Bs, float* C, int M, int N, int K,
                    int G, float alpha, float beta, cudaStream_t st, int prologue, const float* gamma, float eps,
                    const W4Peer* peer, uint32_t* arrivals_out) {
    if (!w4a16_tc_ok(M, N, K, G)) return LHB_ERR_UNSUPPORTED;
    if (arrivals_out) *arrivals_out = 0;
    if (ctx->scratch_bytes < TC_SCRATCH_HEAD) return LHB_ERR_SCRATCH;
    TensorMap tmW;
    if (int e = get_tensor_map_2d_u8(ctx, Bp, K / 2, N, N, TC_ROWS, TC_COLS, false, &tmW)) return e;
    const int mp = tc_slab_rows(M);                         // rows per slab
    const int drows = tc_digit_rows(mp);                    // digit rows per slab
    const size_t slab_bytes = static_cast<size_t>(drows) * K;
    const int slabs_per_pass = std::max<int>(1, std::min<size_t>(1024 / mp, TC_DIG_BYTES / slab_bytes));
    const int rows_per_pass = slabs_per_pass * mp;
    uint8_t* const dig = static_cast<uint8_t*>(ctx->scratch);
    float* const inv = reinterpret_cast<float*>(dig + TC_DIG_BYTES);
    const int S = K / 128, col_tiles = ceil_div(N, TC_COLS);
    const int64_t units = static_cast<int64_t>(S) * col_tiles;
    if (units > (1 << 30) || col_tiles > static_cast<int>(ctx->counters_len)) return LHB_ERR_UNSUPPORTED;
    if (static_cast<int64_t>(mp) * N >= (int64_t(1) << 31)) return LHB_ERR_UNSUPPORTED;
    int ctas = static_cast<int>(std::min<int64_t>(units, ctx->sm_count));
    // A whole number of CTAs per column tile (no CTA straddles two tiles and hands over twice) when
    // that still occupies at least three quarters of the SMs; otherwise an even deal of the units.
    if (col_tiles <= ctas) {
        int per_tile = std::min(S, ctas / col_tiles);
        const int aligned = col_tiles * per_tile;
        if (!knobs().w4tc_stream_k && 4 * aligned >= 3 * ctas) {
            // the kernel takes as long as its longest range: the fewest CTAs per tile with the same longest range
            // mean fewer partial sums to add up (32 units over 8 CTAs instead of 9: 13.1 us instead of 13.9 us)
            while (per_tile > 1 && ceil_div(S, per_tile - 1) == ceil_div(S, per_tile)) --per_tile;
            ctas = col_tiles * per_tile;
        }
    }
    if (knobs().w4tc_ctas > 0) ctas = std::min(ctas, knobs().w4tc_ctas);
    // a whole number (two or more) of CTAs per column tile: the contributors of a tile share its final sum
    const int coop_sum = (knobs().w4tc_coop && ctas % col_tiles == 0 && ctas / col_tiles >= 2 && ctas <= ctx->sm_count) ? 1 : 0;
    const int r_min = std::max<int>(1, static_cast<int>(units / ctas));
    const int max_contrib = std::min(ctas, S / r_min + 2);
    const int64_t row_len = (prologue == TC_PRO_SWIGLU) ? 2 * static_cast<int64_t>(K) : K;
    for (int pass0 = 0; pass0 < M; pass0 += rows_per_pass) {
        const int rows = std::min(rows_per_pass, M - pass0);
        cudaLaunchConfig_t dc = {};
        dc.gridDim = dim3(rows, 1, 1);
        dc.blockDim = dim3(1024, 1, 1);
        dc.stream = st;
        cudaLaunchAttribute da[1];
        da[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        da[0].val.programmaticStreamSerializationAllowed = 1;
        dc.attrs = da;
        dc.numAttrs = tc_pdl() ? 1 : 0;
        LHB_CUDA(cudaLaunchKernelEx(&dc, w4tc_digits_kernel, A + pass0 * row_len, K, mp, reinterpret_cast<int8_t*>(dig),
                                    inv, prologue, gamma, eps));
        const int pass_slabs = ceil_div(rows, mp);
        for (int sl = 0; sl < pass_slabs; ++sl) {
            const int m0 = pass0 + sl * mp, m = std::min(mp, M - m0);
            TensorMap tmD;
            if (int e = get_tensor_map_2d_u8(ctx, dig, static_cast<uint64_t>(pass_slabs) * drows, K, K, drows, 128,
                                             true, &tmD))
                return e;
            if (static_cast<size_t>(col_tiles) * max_contrib * m * TC_COLS * sizeof(float) >
                ctx->scratch_bytes - TC_SCRATCH_HEAD)
                return LHB_ERR_SCRATCH;
            W4TcParams p{};
            p.scales = Bs;
            p.C = C + static_cast<int64_t>(m0) * N;
            p.M = m; p.N = N; p.K = K; p.G = G; p.alpha = alpha; p.beta = beta;
            p.S = S;
            p.units = static_cast<int>(units);
            p.max_contrib = max_contrib;
            p.partial = reinterpret_cast<float*>(dig + TC_SCRATCH_HEAD);
            p.counters = ctx->counters;
            p.coop_sum = coop_sum;
            p.status = ctx->status_word;
            p.inv_scale = inv + (m0 - pass0);
            p.dig_row0 = sl * drows;
            if (peer) {
                p.peer_dst = reinterpret_cast<float* const*>(peer->dst_table);
                p.peer_flags = peer->flag_table;
                p.peer_world = peer->world; p.peer_rank = peer->rank; p.peer_ld = peer->ld; p.peer_col0 = peer->col0;
                p.peer_row0 = m0;
            }
            const int e = peer       ? (mp == 16 ? launch_tc_slab<16, true>(ctx, tmW, tmD, p, ctas, st)
                                                 : launch_tc_slab<32, true>(ctx, tmW, tmD, p, ctas, st))
                          : mp == 16 ? launch_tc_slab<16, false>(ctx, tmW, tmD, p, ctas, st)
                                     : launch_tc_slab<32, false>(ctx, tmW, tmD, p, ctas, st);
            if (e) return e;
            if (peer && arrivals_out) *arrivals_out += static_cast<uint32_t>(col_tiles);   // only launches that will signal
        }
    }
    return LHB_OK;
}

}  // namespace lhb

#ifdef LHB_W4TC_TRACE
extern "C" __attribute__((visibility("default"))) int lhb_debug_w4tc_trace(void* host_out) {
    return static_cast<int>(cudaMemcpyFromSymbol(host_out, lhb::g_tc_trace, sizeof(lhb::g_tc_trace)));
}
#endif

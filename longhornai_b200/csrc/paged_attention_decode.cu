// Split-KV paged decode attention over int8 pages (seq_q == 1).
//
// Pool layout is the reference's: K/V int8 [num_blocks, n_kv_heads, 16, 128]
// with one fp32 scale per (block, head, slot) row
// (src/kernels/kvcache.hpp:34-41, src/kernels/kvcache_quant.hpp:31-36), so a
// page of one head is 2 KiB contiguous for K, 2 KiB for V and 64 B for each
// scale row.  The path is HBM-bound: every page is read once for the whole GQA
// group (up to 4 query heads share a KV head).
//
// Work split: grid = (splits, kv heads, requests).  A CTA owns a contiguous
// range of the request's visible pages; its 4 warps take pages round-robin and
// run independent cp.async rings (3 stages x 4.1 KiB per warp, 128-bit copies,
// XOR-swizzled 16-byte chunks) -- no block-level barrier inside the main loop.
// Per page a warp does, entirely on the int8 tensor-core path (mma.sync s8):
//   S = K Q^T  : m16n8k32, tokens as the 16 rows, head_dim as k; the int8 rows of
//                K are operand registers as they lie in shared memory (no
//                conversion at all); Q is three signed 7-bit digits per element
//                (exact power-of-two scaling per head), one MMA column per digit;
//   softmax in base 2 with the V row scale folded into the exponent:
//                P = 2^(s*c + log2(vs) - m_ref) <= 1 whatever the magnitude of the
//                scales, written as three 7-bit digits of round(2^20 P); the
//                denominator is tracked in fp32 in the same frame;
//   O += V^T P : m16n8k16 with head_dim as the 16 rows and the page's 16 tokens as
//                k; 4x4 byte transposes (byte-permute) turn V rows into operand
//                registers.  The int32 sums stay in the frame of m_ref and are
//                folded into fp32 only when a head's maximum rises above it (the frame is
//                then set 3 above the new maximum, so this happens about once per
//                sequence): the usual page costs no rescaling.
// The four warps merge (m, l, O) in shared memory; with more than one split the
// CTA writes its partial to the context's scratch arena and the last CTA to
// arrive for a (request, kv head) merges the partials in fixed order
// (the (m, l, O) merge rule of flash decoding,
// src/kernels/attention.cpp:255-280 in the reference).
//
// Results differ from the reference's three-pass softmax
// (src/kernels/kvcache_quant.cpp:82-161) only by fp32 summation order and the
// 2^-21 rounding of Q and P to 20-bit integers.

#include <cstdlib>
#include <mutex>
#include <string>

#include "common.cuh"
#include "dispatch.h"

namespace lhb {

// Tuning points (overridable at compile time for experiments)
#ifndef LHB_PD_STAGES
#define LHB_PD_STAGES 4
#endif
#ifndef LHB_PD_MIN_CTAS
#define LHB_PD_MIN_CTAS 3
#endif
constexpr int PD_WARPS = 4;
constexpr int PD_THREADS = PD_WARPS * 32;
constexpr int PD_STAGES = LHB_PD_STAGES;
constexpr int PD_D = 128;
constexpr int PD_BS = 16;
constexpr int PD_STAGE_BYTES = 2048 + 2048 + 64 + 64;          // K, V, ks, vs
constexpr int PD_WARP_BYTES = PD_STAGES * PD_STAGE_BYTES + 256;  // + P digit exchange buffer
constexpr int PD_SMEM_BYTES = PD_WARPS * PD_WARP_BYTES + 2048;  // + the CTA's Q digit fragments
constexpr int PD_MAX_GROUP = 4;
constexpr int PD_PART = PD_D + 2;                               // floats per (split, head): m, l, O[128]
constexpr float PD_WSHIFT = 20.0f;                              // P weights are integers in [0, 2^20]
constexpr float PD_MIN_LOG2_VS = -100.0f;
constexpr float PD_FRAME_MARGIN = 3.0f;                         // head room of the integer frame, in log2 units

__device__ __forceinline__ uint32_t pd_smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Shared-memory accesses by 32-bit shared-space address (no generic 64-bit address math).
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ float ldsf(uint32_t a) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ void sts8(uint32_t a, int v) {
    asm volatile("st.shared.u8 [%0], %1;" ::"r"(a), "r"(v) : "memory");
}
template <int OFF>
__device__ __forceinline__ void cp_async16_off(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1 + %2], 16;" ::"r"(dst), "l"(src), "n"(OFF) : "memory");
}

// int8 x int8 -> int32 tensor-core MMAs (weights / pages as the 16-row operand)
__device__ __forceinline__ void pd_imma32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void pd_imma16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(b0));
}

// exact int32 -> fp32 for |v| < 2^22 without the conversion pipe
__device__ __forceinline__ float pd_i2f(int v) { return __int_as_float(v + 0x4B400000) - 12582912.0f; }

// 4x4 byte transpose: out[b] = {r0.byte b, r1.byte b, r2.byte b, r3.byte b}
__device__ __forceinline__ void pd_transpose4(uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3,
                                              uint32_t (&out)[4]) {
    const uint32_t lo01 = __byte_perm(r0, r1, 0x5140), hi01 = __byte_perm(r0, r1, 0x7362);
    const uint32_t lo23 = __byte_perm(r2, r3, 0x5140), hi23 = __byte_perm(r2, r3, 0x7362);
    out[0] = __byte_perm(lo01, lo23, 0x5410);
    out[1] = __byte_perm(lo01, lo23, 0x7632);
    out[2] = __byte_perm(hi01, hi23, 0x5410);
    out[3] = __byte_perm(hi01, hi23, 0x7632);
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float fast_log2(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

struct DecodeParams {
    const float* Q;          // [n_req, n_q_heads, 1, 128]
    const int8_t* Kp;
    const int8_t* Vp;
    const float* Ks;
    const float* Vs;
    const int32_t* tables;   // [n_req, max_blocks]
    const int32_t* seq_lens; // [n_req]
    float* O;
    float* part;             // scratch: [n_req, n_kv, splits, group, PD_PART]
    int* counters;           // [n_req * n_kv], zero between calls
    int* status;
    int max_blocks, n_q_heads, n_kv_heads, group, num_blocks;
    int splits;              // grid.x: the most splits any request can use
    int pages_per_cta;       // a request is cut into ceil(pages / pages_per_cta) splits, at most `splits`
    int window, chunk;
    float scale_log2e;
};

__global__ void __launch_bounds__(PD_THREADS, LHB_PD_MIN_CTAS)
paged_decode_q8_kernel(const DecodeParams p) {
    extern __shared__ __align__(128) uint8_t pd_smem[];
    __shared__ int s_last;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int split = blockIdx.x, kvh = blockIdx.y, req = blockIdx.z;
    const int G = p.group;

    // ---- visible key range of the single query row (seq_q == 1) -------------
    int len = p.seq_lens[req];
    len = max(0, min(len, p.max_blocks * PD_BS));
    const int last = len - 1;
    int first = 0;
    if (p.window > 0) first = max(0, len - p.window);
    if (p.chunk > 0 && len > 0) first = max(first, (last / p.chunk) * p.chunk);
    const int page_f = first / PD_BS;
    const int n_pages = (len > 0 && last >= first) ? last / PD_BS - page_f + 1 : 0;
    // Long requests are cut into more pieces than short ones, so that every CTA
    // has about the same number of pages; CTAs beyond a request's piece count leave.
    const int nsplit = max(1, min(p.splits, (n_pages + p.pages_per_cta - 1) / p.pages_per_cta));
    if (split >= nsplit) return;
    const int per_split = (n_pages + nsplit - 1) / nsplit;
    const int pg_lo = page_f + split * per_split;
    const int pg_hi = min(page_f + n_pages, pg_lo + per_split);   // exclusive
    const int32_t* table = p.tables + static_cast<int64_t>(req) * p.max_blocks;

    // ---- Q as three signed 7-bit digits per element (q*s = d1*2^14 + d2*2^7 + d3, s a
    // power of two per head putting max|q| in [2^19, 2^20)), one int8 MMA column per
    // digit.  Column layout of the two 8-column operand blocks: block 0 column 2h = d1,
    // 2h+1 = d2 of head h; block 1 column 2h = d3 (odd columns zero), so thread (g, t)
    // of the result fragment owns every digit of head t.  Thread (g, t) of the operand
    // holds column g at head_dim positions 32t + 8i .. +7 for k-step i.
    const int hq = g >> 1, odd = g & 1;
    uint32_t qf[4][2][2];            // [k-step][block][register]
    float qinv[PD_MAX_GROUP];
    {
        const float* qbase = p.Q + (static_cast<int64_t>(req) * p.n_q_heads + kvh * G) * PD_D;
#pragma unroll
        for (int h = 0; h < PD_MAX_GROUP; ++h) {
            float mx = 0.0f;
            if (h < G) {
                const float4 v = *reinterpret_cast<const float4*>(qbase + h * PD_D + lane * 4);
                mx = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
            }
            mx = warp_max(mx);
            const int e = static_cast<int>((__float_as_uint(mx) >> 23) & 0xff);
            int se = (mx > 0.0f) ? 273 - e : 127;          // 127 + 19 - (e - 127)
            se = max(1, min(253, se));
            qinv[h] = __uint_as_float(static_cast<uint32_t>(254 - se) << 23);
        }
        float qs = 0.0f;
#pragma unroll
        for (int h = 0; h < PD_MAX_GROUP; ++h)
            if (h == hq) qs = 1.0f / qinv[h];          // exact: powers of two
        const bool live = hq < G;
        // warp w converts k-step w; the CTA shares the fragments through shared memory
        uint32_t* qsm = reinterpret_cast<uint32_t*>(pd_smem + PD_WARPS * PD_WARP_BYTES);    // [k-step][block][reg][lane]
        {
            const int i = warp;
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (live) v = *reinterpret_cast<const float4*>(qbase + hq * PD_D + 32 * t + 8 * i + 4 * r);
                const float x[4] = {v.x * qs, v.y * qs, v.z * qs, v.w * qs};
                uint32_t b0 = 0, b1 = 0;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    int iv = __float2int_rn(fminf(fmaxf(x[j], -1048576.0f), 1048576.0f));
                    const int lo = ((iv + 64) & 127) - 64;
                    iv = (iv - lo) >> 7;
                    const int mid = ((iv + 64) & 127) - 64;
                    const int hi = (iv - mid) >> 7;
                    b0 |= static_cast<uint32_t>((odd ? mid : hi) & 0xff) << (8 * j);
                    b1 |= static_cast<uint32_t>((odd ? 0 : lo) & 0xff) << (8 * j);
                }
                qsm[((i * 2 + 0) * 2 + r) * 32 + lane] = b0;
                qsm[((i * 2 + 1) * 2 + r) * 32 + lane] = b1;
            }
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int b = 0; b < 2; ++b)
#pragma unroll
                for (int r = 0; r < 2; ++r) qf[i][b][r] = qsm[((i * 2 + b) * 2 + r) * 32 + lane];
    }

    // ---- per-warp state ---------------------------------------------------------
    uint8_t* ring = pd_smem + warp * PD_WARP_BYTES;
    const uint32_t ring_u32 = pd_smem_u32(ring);
    uint8_t* pdig = ring + PD_STAGES * PD_STAGE_BYTES;   // [2 blocks][8 columns][16 tokens] digit bytes of P
    for (int i = lane; i < 64; i += 32) reinterpret_cast<uint32_t*>(pdig)[i] = 0u;             // odd columns of block 1 stay zero
    __syncwarp();
    int oi0[8][4], oi1[8][4];        // int32 sums of V^T P since the last fold: block 0 (d1, d2), block 1 (d3)
    float of[8][2];                  // folded fp32 output of head t at head_dim 16g + i and 16g + 8 + i
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        oi0[i][0] = oi0[i][1] = oi0[i][2] = oi0[i][3] = 0;
        oi1[i][0] = oi1[i][1] = oi1[i][2] = oi1[i][3] = 0;
        of[i][0] = of[i][1] = 0.0f;
    }
    float m_ref = -INFINITY;      // reference exponent of head t (identical on the 8 lanes that share t)
    float l_run = 0.0f;           // this lane's share of the denominator, in the frame of m_ref
    int pages_since_fold = 0;
    const float sc = p.scale_log2e * (t == 0 ? qinv[0] : t == 1 ? qinv[1] : t == 2 ? qinv[2] : qinv[3]);

    // Fold the int32 sums (taken in the frame of the current m_ref) into the fp32
    // output, move both to a new frame by `alpha`, and clear the sums.
    auto fold = [&](float alpha) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float a = fmaf(16384.0f, __int2float_rn(oi0[i][0]),
                                 fmaf(128.0f, __int2float_rn(oi0[i][1]), __int2float_rn(oi1[i][0])));
            const float b = fmaf(16384.0f, __int2float_rn(oi0[i][2]),
                                 fmaf(128.0f, __int2float_rn(oi0[i][3]), __int2float_rn(oi1[i][2])));
            of[i][0] = (of[i][0] + a) * alpha;
            of[i][1] = (of[i][1] + b) * alpha;
            oi0[i][0] = oi0[i][1] = oi0[i][2] = oi0[i][3] = 0;
            oi1[i][0] = oi1[i][1] = oi1[i][2] = oi1[i][3] = 0;
        }
    };

    const int my_first = pg_lo + warp;                 // this warp's pages: my_first, +4, +8, ...
    const int n_iter = (pg_hi > my_first) ? (pg_hi - my_first + PD_WARPS - 1) / PD_WARPS : 0;

    // Page ids: lane l of `ids` holds the id of iteration 32*batch + l of the batch the
    // prefetcher is in; validity of the pages in flight is remembered in `ok_bits`.
    int32_t ids = 0;
    int ids_batch = -1;
    uint32_t ok_bits = 0;                               // bit (it & 31): page of iteration it is valid
    // lane-constant pieces of the page copy: 16-byte chunk idx = c*32 + lane of a 2 KiB page goes to
    // token idx/8, chunk (idx%8) ^ (token%8); for c the token is 4c + lane/8
    const uint32_t cp_d0 = (lane >> 3) * 128 + (((lane & 7) ^ (lane >> 3)) << 4);
    const uint32_t lane16 = lane * 16;
    uint32_t issue_off = 0;                             // stage offset of the next copy in the ring
    auto issue = [&](int it) {
        if (it < n_iter) {
            if ((it >> 5) != ids_batch) {               // entering a new batch of 32 iterations
                ids_batch = it >> 5;
                const int j = ids_batch * 32 + lane;
                ids = (j < n_iter) ? table[my_first + j * PD_WARPS] : 0;
            }
            int blk = __shfl_sync(0xffffffffu, ids, it & 31);
            const bool okp = blk >= 0 && blk < p.num_blocks;
            ok_bits = okp ? (ok_bits | (1u << (it & 31))) : (ok_bits & ~(1u << (it & 31)));
            if (!okp) blk = 0;                          // masked at use; a bad id is never dereferenced
            const int64_t row0 = (static_cast<int64_t>(blk) * p.n_kv_heads + kvh) * PD_BS;
            const uint32_t st = ring_u32 + issue_off;
            const int8_t* kp = p.Kp + row0 * PD_D + lane16;
            const int8_t* vp = p.Vp + row0 * PD_D + lane16;
            // tokens 4c + lane/8: sw differs from sw(lane/8) by (c & 1) << 2 and (c >> 1) << 1
            const uint32_t d0 = st + cp_d0, d1 = st + (cp_d0 ^ 64), d2 = st + (cp_d0 ^ 32), d3 = st + (cp_d0 ^ 96);
            cp_async16_off<0>(d0, kp);            cp_async16_off<0>(d0 + 2048, vp);
            cp_async16_off<512>(d1 + 512, kp);    cp_async16_off<512>(d1 + 2048 + 512, vp);
            cp_async16_off<1024>(d2 + 1024, kp);  cp_async16_off<1024>(d2 + 2048 + 1024, vp);
            cp_async16_off<1536>(d3 + 1536, kp);  cp_async16_off<1536>(d3 + 2048 + 1536, vp);
            if (lane < 4) cp_async16(st + 4096 + lane16, p.Ks + row0 + lane * 4);
            else if (lane < 8) cp_async16(st + 4160 + lane16 - 64, p.Vs + row0 + (lane - 4) * 4);
        }
        issue_off = (issue_off == (PD_STAGES - 1) * PD_STAGE_BYTES) ? 0 : issue_off + PD_STAGE_BYTES;
        cp_async_commit();
    };

#pragma unroll
    for (int s = 0; s < PD_STAGES - 1; ++s) issue(s);

    // lane-constant shared offsets inside a stage
    // 16-byte chunk c of token row r sits at chunk c ^ sw(r), sw(r) = (r & 5) | (((r >> 1) ^ (r >> 3)) & 1) << 1:
    // conflict-free for the K reads (rows g, g+8) and the V reads (rows 4t + j) alike
    const uint32_t ka = g * 128 + (((2 * t) ^ g) << 4);                 // K: token g, chunk 2t (chunk 2t+1: ^16; token g+8: (^32) + 1024)
    const uint32_t vb = 2048 + 4 * t * 128 + ((g ^ ((t >> 1) << 1) ^ ((t & 1) << 2)) << 4);  // V: token 4t + j: (vb ^ (j << 4)) + 128 j
    const uint32_t pdig_u32 = ring_u32 + PD_STAGES * PD_STAGE_BYTES;
    const uint32_t pst = pdig_u32 + 32 * t + g;                         // digit bytes of this thread's tokens g, g+8
    const uint32_t pld = pdig_u32 + g * 16 + 4 * t;                     // operand register: column g, tokens 4t..4t+3
    uint32_t use_off = 0;

    for (int it = 0; it < n_iter; ++it) {
        cp_async_wait<PD_STAGES - 2>();
        __syncwarp();                                   // every lane is done with iteration it - 1
        issue(it + PD_STAGES - 1);                      // refills the stage iteration it - 1 used
        const uint32_t st = ring_u32 + use_off;
        use_off = (use_off == (PD_STAGES - 1) * PD_STAGE_BYTES) ? 0 : use_off + PD_STAGE_BYTES;
        const int tok0 = (my_first + it * PD_WARPS) * PD_BS;
        const bool page_ok = (ok_bits >> (it & 31)) & 1u;

        // ---- S = K Q^T: int8 rows of K are MMA operand registers as they lie ------------
        int s0[4] = {0, 0, 0, 0}, s1[4] = {0, 0, 0, 0};     // block 0: (d1, d2) of head t; block 1: d3
        {
            const uint4 a0 = lds128(st + ka), a1 = lds128(st + (ka ^ 16));                   // token g
            const uint4 b0 = lds128(st + (ka ^ 32) + 1024), b1 = lds128(st + (ka ^ 48) + 1024);   // token g + 8
            const uint32_t wa[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const uint32_t wb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                pd_imma32(s0, wa[2 * i], wb[2 * i], wa[2 * i + 1], wb[2 * i + 1], qf[i][0][0], qf[i][0][1]);
                pd_imma32(s1, wa[2 * i], wb[2 * i], wa[2 * i + 1], wb[2 * i + 1], qf[i][1][0], qf[i][1][1]);
            }
        }
        // ---- scores in base 2, V row scale folded into the exponent ------------------------
        const uint32_t sca = st + 4096 + 4 * g;               // ks[g], +32: ks[g+8], +64: vs[g], +96: vs[g+8]
        float x0 = fmaf(16384.0f, pd_i2f(s0[0]), fmaf(128.0f, pd_i2f(s0[1]), pd_i2f(s1[0]))) * ldsf(sca) * sc;
        float x1 = fmaf(16384.0f, pd_i2f(s0[2]), fmaf(128.0f, pd_i2f(s0[3]), pd_i2f(s1[2]))) * ldsf(sca + 32) * sc;
        const int p0 = tok0 + g, p1 = tok0 + g + 8;
        const bool ok0 = page_ok && p0 >= first && p0 <= last;
        const bool ok1 = page_ok && p1 >= first && p1 <= last;
        const float lv0 = fmaxf(fast_log2(ldsf(sca + 64)), PD_MIN_LOG2_VS);
        const float lv1 = fmaxf(fast_log2(ldsf(sca + 96)), PD_MIN_LOG2_VS);
        x0 = ok0 ? x0 : -INFINITY;
        x1 = ok1 ? x1 : -INFINITY;
        const float y0 = x0 + lv0, y1 = x1 + lv1;              // -inf stays -inf
        float mp = fmaxf(y0, y1);
        mp = fmaxf(mp, __shfl_xor_sync(0xffffffffu, mp, 4));
        mp = fmaxf(mp, __shfl_xor_sync(0xffffffffu, mp, 8));
        mp = fmaxf(mp, __shfl_xor_sync(0xffffffffu, mp, 16));
        // The int32 sums are kept in the frame of m_ref.  When a head's maximum rises
        // above it, the sums are folded into fp32 and the frame moves to the new
        // maximum plus a margin of 3 (weights then start at <= 2^-3 of full scale,
        // still 17 bits), so that later, smaller rises need no fold; a sequence
        // usually folds once.  Every 4096 pages a fold keeps the int32 sums in range.
        const bool rise = mp > m_ref;
        if (__any_sync(0xffffffffu, rise) || pages_since_fold == 4096) {
            const float m_new = rise ? mp + PD_FRAME_MARGIN : m_ref;
            const float alpha = (m_new == m_ref) ? 1.0f : fast_exp2(m_ref - m_new);   // exp2(-inf) = 0
            fold(alpha);
            l_run *= alpha;
            m_ref = m_new;
            pages_since_fold = 0;
        }
        ++pages_since_fold;
        const float mb = (m_ref == -INFINITY) ? 0.0f : m_ref;
        l_run += fast_exp2(x0 - mb) + fast_exp2(x1 - mb);
        // ---- P = 2^20 * 2^(y - m_ref) <= 2^20 as three 7-bit digits, through shared memory
        // into operand order: column c of a block, tokens 4t .. 4t+3 in one register
        {
            int w0 = __float2int_rn(fast_exp2(y0 - mb + PD_WSHIFT));
            int w1 = __float2int_rn(fast_exp2(y1 - mb + PD_WSHIFT));
            const int l0 = ((w0 + 64) & 127) - 64; w0 = (w0 - l0) >> 7;
            const int l1 = ((w1 + 64) & 127) - 64; w1 = (w1 - l1) >> 7;
            const int m0 = ((w0 + 64) & 127) - 64; const int h0 = (w0 - m0) >> 7;
            const int m1 = ((w1 + 64) & 127) - 64; const int h1 = (w1 - m1) >> 7;
            // block 0 column 2t (d1) at +0, column 2t+1 (d2) at +16, block 1 column 2t (d3) at +128
            sts8(pst, h0); sts8(pst + 8, h1);
            sts8(pst + 16, m0); sts8(pst + 24, m1);
            sts8(pst + 128, l0); sts8(pst + 136, l1);
        }
        __syncwarp();
        const uint32_t pb0 = lds32(pld);
        const uint32_t pb1 = lds32(pld + 128);
        // ---- O += V^T P: 4x4 byte transposes turn V rows into "4 tokens of one head_dim" registers
        {
            uint32_t vr[4][4];                          // [token 4t + j][word: head_dim 16g + 4w .. +3]
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint4 v = lds128(st + ((vb ^ (j << 4)) + 128 * j));
                vr[j][0] = v.x; vr[j][1] = v.y; vr[j][2] = v.z; vr[j][3] = v.w;
            }
#pragma unroll
            for (int w = 0; w < 2; ++w) {
                // head_dim 16g + 4w + b (operand row g) and 16g + 8 + 4w + b (row g + 8), b = 0..3
                uint32_t ta[4], tb[4];
                pd_transpose4(vr[0][w], vr[1][w], vr[2][w], vr[3][w], ta);
                pd_transpose4(vr[0][w + 2], vr[1][w + 2], vr[2][w + 2], vr[3][w + 2], tb);
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    pd_imma16(oi0[4 * w + b], ta[b], tb[b], pb0);
                    pd_imma16(oi1[4 * w + b], ta[b], tb[b], pb1);
                }
            }
        }
    }
    cp_async_wait<0>();
    fold(1.0f);

    // ---- merge the four warps in shared memory -------------------------------------------
    __syncthreads();                                   // rings are dead from here on
    float* sm_m = reinterpret_cast<float*>(pd_smem);                   // [4 warps][4 heads]
    float* sm_l = sm_m + PD_WARPS * PD_MAX_GROUP;                      // [4][4]
    float* sm_o = sm_l + PD_WARPS * PD_MAX_GROUP;                      // [4 warps][4 heads][128]
    {
        float l = l_run;
        l += __shfl_xor_sync(0xffffffffu, l, 4);
        l += __shfl_xor_sync(0xffffffffu, l, 8);
        l += __shfl_xor_sync(0xffffffffu, l, 16);
        if (g == 0) { sm_m[warp * PD_MAX_GROUP + t] = m_ref; sm_l[warp * PD_MAX_GROUP + t] = l; }
        float* od = sm_o + (warp * PD_MAX_GROUP + t) * PD_D + 16 * g;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            od[i] = of[i][0];
            od[8 + i] = of[i][1];
        }
    }
    __syncthreads();
    const int d = threadIdx.x;                          // 128 threads <-> 128 head_dim elements
    const int64_t pbase = ((static_cast<int64_t>(req) * p.n_kv_heads + kvh) * p.splits + split) * G;
    for (int h = 0; h < G; ++h) {
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < PD_WARPS; ++w) M = fmaxf(M, sm_m[w * PD_MAX_GROUP + h]);
        float L = 0.0f, o = 0.0f;
#pragma unroll
        for (int w = 0; w < PD_WARPS; ++w) {
            const float mw = sm_m[w * PD_MAX_GROUP + h];
            const float f = (mw == -INFINITY) ? 0.0f : fast_exp2(mw - M);
            L += f * sm_l[w * PD_MAX_GROUP + h];
            o += f * sm_o[(w * PD_MAX_GROUP + h) * PD_D + d];
        }
        if (nsplit == 1) {
            float* out = p.O + (static_cast<int64_t>(req) * p.n_q_heads + kvh * G + h) * PD_D;
            out[d] = (L > 0.0f) ? o * (1.0f / L) * exp2f(-PD_WSHIFT) : 0.0f;
        } else {
            float* pp = p.part + (pbase + h) * PD_PART;
            if (d == 0) { pp[0] = M; pp[1] = L; }
            pp[2 + d] = o;
        }
    }
    if (nsplit == 1) return;

    // ---- cross-CTA merge: the last split to arrive combines all partials ------------------
    // One thread fences for the CTA on either side of the count: the barrier before it
    // orders every thread's partial stores ahead of the fence, the barrier after it orders
    // the other splits' stores ahead of every thread's loads.
    __syncthreads();
    const int cidx = req * p.n_kv_heads + kvh;
    if (threadIdx.x == 0) {
        __threadfence();
        const int old = atomicAdd(p.counters + cidx, 1);
        s_last = (old == nsplit - 1);
        if (s_last) {
            p.counters[cidx] = 0;                      // ready for the next call
            __threadfence();                           // only the merging CTA reads the others' stores
        }
    }
    __syncthreads();
    if (!s_last) return;
    // One warp per query head, a lane per four output dimensions; the partials of up to
    // eight splits are in flight together, so the merge costs one memory round trip per
    // eight splits instead of one per partial.  Splits are folded in split order with a
    // running maximum (deterministic).
    const int64_t b0 = (static_cast<int64_t>(req) * p.n_kv_heads + kvh) * p.splits * G;
    const int mw = threadIdx.x >> 5, ml = threadIdx.x & 31;
    for (int h = mw; h < G; h += PD_WARPS) {
        float M = -INFINITY, L = 0.0f;
        float2 oa = make_float2(0.f, 0.f), ob = make_float2(0.f, 0.f);   // dims 2*ml.. and 64 + 2*ml..
        for (int s0 = 0; s0 < nsplit; s0 += 8) {
            float ms[8], ls[8];
            float2 va[8], vb[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                ms[j] = -INFINITY; ls[j] = 0.0f;
                va[j] = make_float2(0.f, 0.f); vb[j] = make_float2(0.f, 0.f);
                if (s0 + j < nsplit) {
                    const float* pp = p.part + (b0 + (s0 + j) * G + h) * PD_PART;
                    ms[j] = __ldcg(pp);
                    ls[j] = __ldcg(pp + 1);
                    va[j] = __ldcg(reinterpret_cast<const float2*>(pp + 2 + 2 * ml));
                    vb[j] = __ldcg(reinterpret_cast<const float2*>(pp + 2 + 64 + 2 * ml));
                }
            }
            float Mb = M;
#pragma unroll
            for (int j = 0; j < 8; ++j) Mb = fmaxf(Mb, ms[j]);
            const float keep = (M == -INFINITY) ? 0.0f : fast_exp2(M - Mb);
            L *= keep; oa.x *= keep; oa.y *= keep; ob.x *= keep; ob.y *= keep;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float f = (ms[j] == -INFINITY) ? 0.0f : fast_exp2(ms[j] - Mb);
                L += f * ls[j];
                oa.x += f * va[j].x; oa.y += f * va[j].y;
                ob.x += f * vb[j].x; ob.y += f * vb[j].y;
            }
            M = Mb;
        }
        float* out = p.O + (static_cast<int64_t>(req) * p.n_q_heads + kvh * G + h) * PD_D;
        const float r = (L > 0.0f) ? (1.0f / L) * exp2f(-PD_WSHIFT) : 0.0f;
        *reinterpret_cast<float2*>(out + 2 * ml) = make_float2(oa.x * r, oa.y * r);
        *reinterpret_cast<float2*>(out + 64 + 2 * ml) = make_float2(ob.x * r, ob.y * r);
    }
}

// How a request is cut: the longest request the table can describe is cut into `splits`
// equal pieces of `pages` pages (16 tokens each); shorter requests use fewer pieces.  Sized
// so that about four CTAs per SM (an SM holds three at a time) would exist if every
// request were as long as the table, within 16..128 pages per CTA (fewer pages: the per-CTA
// set-up dominates; more: the last CTAs to finish leave SMs idle).
static void decode_split_plan(int sm_count, int64_t items, int max_blocks, size_t part_floats_avail, int group,
                              int* splits, int* pages) {
    int target = 4;                                          // CTAs per SM if every request were as long as the table
    if (knobs().decode_target > 0) target = knobs().decode_target;
    int64_t pp = items * max_blocks / (static_cast<int64_t>(target) * std::max(1, sm_count));
    int pg = static_cast<int>(std::max<int64_t>(16, std::min<int64_t>(128, pp)));
    if (knobs().decode_pages > 0) pg = knobs().decode_pages;
    int sp = std::max(1, std::min(32, ceil_div(max_blocks, pg)));
    // When all (request, KV head) items fit the resident CTA slots, one wave of the longest pieces that still
    // fills the slots beats more, shorter pieces in a second wave (32 requests x 8 heads x 129 pages: 31.4 us as
    // 256 CTAs, 37.5 us as 768, 44.7 us as 512).
    const int64_t slots = static_cast<int64_t>(LHB_PD_MIN_CTAS) * std::max(1, sm_count);
    if (knobs().decode_one_wave && knobs().decode_pages == 0 && knobs().decode_target == 0 && items <= slots)
        sp = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(std::min<int64_t>(32, slots / items), max_blocks / 16)));
    if (knobs().decode_splits > 0) sp = std::min(sp, knobs().decode_splits);
    const size_t per_split = static_cast<size_t>(items) * group * PD_PART;
    if (sp > 1 && per_split * sp > part_floats_avail)
        sp = static_cast<int>(std::max<size_t>(1, part_floats_avail / per_split));
    *splits = sp;
    *pages = ceil_div(max_blocks, sp);      // equal pieces of the longest request; covers every page of it
}

bool decode_fast_ok(const lhb_paged_attn_cfg& cfg, const lhb_paged_layout& L) {
    if (cfg.seq_q != 1 || cfg.head_dim != PD_D || L.head_dim != PD_D || L.block_size != PD_BS) return false;
    if (cfg.n_kv_heads <= 0 || cfg.n_q_heads % cfg.n_kv_heads) return false;
    const int group = cfg.n_q_heads / cfg.n_kv_heads;
    return group >= 1 && group <= PD_MAX_GROUP && cfg.n_kv_heads <= 65535;
}

int launch_decode_fast(lhb_ctx* ctx, const float* Q, const int8_t* Kp, const int8_t* Vp,
                       const float* Ks, const float* Vs, const int32_t* tables, int max_blocks,
                       const int32_t* seq_lens, int n_req, float* O, const lhb_paged_attn_cfg& cfg,
                       const lhb_paged_layout& L, cudaStream_t st) {
    const int group = cfg.n_q_heads / cfg.n_kv_heads;
    const int64_t items = static_cast<int64_t>(n_req) * cfg.n_kv_heads;
    int splits = 1, pages = max_blocks;
    decode_split_plan(ctx->sm_count, items, max_blocks,
                      items > static_cast<int64_t>(ctx->counters_len) ? 0 : ctx->scratch_bytes / sizeof(float), group,
                      &splits, &pages);
    DecodeParams p{};
    p.Q = Q; p.Kp = Kp; p.Vp = Vp; p.Ks = Ks; p.Vs = Vs; p.tables = tables; p.seq_lens = seq_lens;
    p.O = O; p.part = reinterpret_cast<float*>(ctx->scratch); p.counters = ctx->counters;
    p.status = ctx->status_word;
    p.max_blocks = max_blocks; p.n_q_heads = cfg.n_q_heads; p.n_kv_heads = cfg.n_kv_heads;
    p.group = group; p.num_blocks = L.num_blocks; p.splits = splits; p.pages_per_cta = pages;
    p.window = cfg.window; p.chunk = cfg.chunk;
    const float scale = cfg.scale > 0.0f ? cfg.scale : 1.0f / sqrtf(static_cast<float>(cfg.head_dim));
    p.scale_log2e = scale * 1.4426950408889634f;
    const size_t smem = PD_SMEM_BYTES;
    static bool attr_set[64] = {};
    if (!attr_set[ctx->device & 63]) {
        LHB_CUDA(cudaFuncSetAttribute(paged_decode_q8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(smem)));
        attr_set[ctx->device & 63] = true;
    }
    dim3 grid(splits, cfg.n_kv_heads, n_req);
    paged_decode_q8_kernel<<<grid, PD_THREADS, smem, st>>>(p);
    LHB_LAUNCH_CHECK();
    return LHB_OK;
}

// ---------------------------------------------------------------------------
// Decode attention for callers that must not allocate device memory.
//
// Some hosts cannot give this library a context, because creating one calls
// cudaMalloc: a serving process that has already handed every free byte of HBM
// to its own KV pools, a plugin loaded into a host whose rules forbid
// allocation after start-up, or a latency-critical loop that cannot afford the
// device-wide synchronisation an allocation may imply.  For them the split-KV
// partials, the arrival counters and the status word of the kernel above live
// in fixed arrays inside the library image instead of a context's arena.
//
// Limits (checked, reported as LHB_ERR_SCRATCH with a message):
//   n_requests * n_kv_heads                          <= 4096  (one counter each)
//   n_requests * n_kv_heads * splits * group * 130 floats <= 8 MiB of partials
// Every GPU that loads the library holds these arrays (about 8 MiB) until the
// process exits.  All calls on a device share them and they keep the previous
// call's contents: the counters are cleared on the stream at the start of each
// call, the partials are always written before they are read.  Two calls that
// overlap on the GPU (different streams) race on the arrays; serialise them.
// ---------------------------------------------------------------------------

constexpr size_t NA_PART_FLOATS = (size_t(8) << 20) / sizeof(float);
constexpr int NA_COUNTERS = 4096;

static __device__ __align__(256) float g_na_partials[NA_PART_FLOATS];
static __device__ __align__(256) int g_na_counters[NA_COUNTERS];
static __device__ __align__(256) int g_na_status[64];

namespace {

struct NoAllocDevice {
    float* partials = nullptr;     // device addresses of the arrays above on this device
    int* counters = nullptr;
    int* status = nullptr;
    int sm_count = 0;
    bool ready = false;
};

std::mutex g_na_mu;
NoAllocDevice g_na_dev[64];

// Once per device, with that device current: in host code the array names are
// only handles, the addresses a kernel can use come from cudaGetSymbolAddress.
int na_setup(int dev, NoAllocDevice** out) {
    std::lock_guard<std::mutex> lk(g_na_mu);
    NoAllocDevice& d = g_na_dev[dev & 63];
    if (!d.ready) {
        LHB_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&d.partials), g_na_partials));
        LHB_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&d.counters), g_na_counters));
        LHB_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&d.status), g_na_status));
        LHB_CUDA(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
        LHB_CUDA(cudaFuncSetAttribute(paged_decode_q8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      PD_SMEM_BYTES));
        d.ready = true;
    }
    *out = &d;
    return LHB_OK;
}

}  // namespace
}  // namespace lhb

extern "C" int lhb_paged_attention_q8_batched_noalloc(
    const float* Q, const int8_t* K_pool, const int8_t* V_pool, const float* K_scales,
    const float* V_scales, const int32_t* block_tables, int max_blocks_per_req,
    const int32_t* seq_lens, int n_requests, float* O, const lhb_paged_attn_cfg* cfg,
    const lhb_paged_layout* layout, void* stream) {
    using namespace lhb;
    if (!Q || !K_pool || !V_pool || !K_scales || !V_scales || !block_tables || !seq_lens || !O || !cfg || !layout)
        return LHB_ERR_NULL;
    if (n_requests < 0 || n_requests > 65535 || max_blocks_per_req <= 0 || layout->num_blocks <= 0)
        return LHB_ERR_BAD_SHAPE;
    if (cfg->head_dim != layout->head_dim || cfg->n_kv_heads != layout->n_kv_heads || cfg->window < 0 ||
        cfg->chunk < 0 || cfg->n_q_heads <= 0)
        return LHB_ERR_BAD_SHAPE;
    if (!decode_fast_ok(*cfg, *layout)) {
        set_last_error_text("lhb_paged_attention_q8_batched_noalloc: only the decode shape is served "
                            "(seq_q 1, head_dim 128, block_size 16, at most 4 query heads per KV head)");
        return LHB_ERR_UNSUPPORTED;
    }
    if (!aligned16(Q) || !aligned16(K_pool) || !aligned16(V_pool) || !aligned16(K_scales) ||
        !aligned16(V_scales) || !aligned16(O))
        return LHB_ERR_MISALIGNED;
    if (n_requests == 0) return LHB_OK;
    int dev = 0;
    LHB_CUDA(cudaGetDevice(&dev));
    NoAllocDevice* d = nullptr;
    if (int e = na_setup(dev, &d)) return e;

    const int group = cfg->n_q_heads / cfg->n_kv_heads;
    const int64_t items = static_cast<int64_t>(n_requests) * cfg->n_kv_heads;
    if (items > NA_COUNTERS) {
        set_last_error_text("lhb_paged_attention_q8_batched_noalloc: n_requests * n_kv_heads = " +
                            std::to_string(items) + " exceeds the fixed limit of " + std::to_string(NA_COUNTERS));
        return LHB_ERR_SCRATCH;
    }
    // same split rule as the context-based entry point with its default arena, so both give the same bits
    int splits = 1, pages = max_blocks_per_req;
    decode_split_plan(d->sm_count, items, max_blocks_per_req, size_t(64) << 18, group, &splits, &pages);
    const size_t need = static_cast<size_t>(items) * splits * group * PD_PART;
    if (splits > 1 && need > NA_PART_FLOATS) {
        set_last_error_text("lhb_paged_attention_q8_batched_noalloc: " + std::to_string(need * sizeof(float)) +
                            " bytes of split partials exceed the fixed 8 MiB array");
        return LHB_ERR_SCRATCH;
    }
    cudaStream_t st = as_stream(stream);
    LHB_CUDA(cudaMemsetAsync(d->counters, 0, sizeof(int) * static_cast<size_t>(items), st));

    DecodeParams p{};
    p.Q = Q; p.Kp = K_pool; p.Vp = V_pool; p.Ks = K_scales; p.Vs = V_scales;
    p.tables = block_tables; p.seq_lens = seq_lens; p.O = O;
    p.part = d->partials; p.counters = d->counters; p.status = d->status;
    p.max_blocks = max_blocks_per_req; p.n_q_heads = cfg->n_q_heads; p.n_kv_heads = cfg->n_kv_heads;
    p.group = group; p.num_blocks = layout->num_blocks; p.splits = splits; p.pages_per_cta = pages;
    p.window = cfg->window; p.chunk = cfg->chunk;
    const float scale = cfg->scale > 0.0f ? cfg->scale : 1.0f / sqrtf(static_cast<float>(cfg->head_dim));
    p.scale_log2e = scale * 1.4426950408889634f;
    dim3 grid(splits, cfg->n_kv_heads, n_requests);
    paged_decode_q8_kernel<<<grid, PD_THREADS, PD_SMEM_BYTES, st>>>(p);
    LHB_LAUNCH_CHECK();
    return LHB_OK;
}

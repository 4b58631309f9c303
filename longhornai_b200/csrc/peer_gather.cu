// Exchange step of the tensor-parallel decode layer over NVLink peer memory.
//
// The reference is single-device (src/runtime/scheduler.hpp:47 drives one
// model on one host), so there is no reference interface behind this file: it
// is the one place where the sharded step of this library has to move data
// between GPUs.  Each rank owns a column slab [rows, width] of an activation
// and every rank needs the whole row-major [rows, world*width] matrix before
// its next GEMM.  The tensors are 16..900 KB, so the cost of a library
// all-gather is its launch and rendezvous latency, not bandwidth; here one
// launch per rank PUSHES the slab straight into its final place in every
// peer's buffer with plain 16-byte stores, then raises a counter in the
// peer's memory, and waits until its own counters show that every peer's slab
// has landed.  No staging buffer, no second copy to re-lay the slabs out.
//
// Protocol.  Rank r keeps `arrivals[world]` (uint32, in peer-visible memory)
// and a private `state[4]` = {expected, tickets, status, unused}.  A call with
// `cpp` CTAs per peer adds cpp to arrivals[r] of every peer (one
// red.release.sys per CTA, after its stores); the call is complete on rank r
// when every arrivals[p] has reached state.expected + cpp.  Counters only grow
// (wrap-safe comparison), so calls need no reset and no host round trip, and
// the launch can sit in a CUDA graph.  Every rank must issue the same sequence
// of calls with the same shapes.  A rank can run at most one call ahead of a
// peer (its next wait needs that peer's next push), so consecutive calls must
// target different destination buffers, and a destination must not be read
// between the call before it and the call that fills it.
//
// Every wait is bounded: after `timeout_ms` the waiting thread records
// 1 + the silent peer in state.status and the kernel returns; the host reads
// it with lhb_peer_status.  CTAs push before they wait and wait only on other
// GPUs, so no scheduling order of the grid can deadlock it.
#include "common.cuh"
#include "dispatch.h"

namespace lhb {

__device__ __forceinline__ unsigned long long pg_now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void pg_signal(uint32_t* counter) {
    asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(counter) : "memory");
}

__device__ __forceinline__ uint32_t pg_peek(const uint32_t* counter) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
    return v;
}

// grid = world * cpp CTAs.  CTA (p, c) copies every cpp-th 16-byte piece of the
// local slab to peer (rank + p) % world, signals it, and (c == 0) waits for
// that peer's slab to arrive here.
__global__ void __launch_bounds__(512)
peer_allgather_cols_kernel(const float4* __restrict__ local, int rows, int w4, float4* const* __restrict__ dst_table,
                           uint32_t* const* __restrict__ flag_table, uint32_t* __restrict__ state, int rank, int world,
                           int cpp, unsigned long long timeout_ns) {
    const int p = blockIdx.x / cpp, c = blockIdx.x - p * cpp;
    const int peer = (rank + p) % world;
    // every CTA reads the expected count before any CTA can advance it: the
    // advance is made by the CTA that takes the last ticket, at its very end
    const uint32_t target = state[0] + static_cast<uint32_t>(cpp);
    float4* dst = dst_table[peer];
    const int total = rows * w4;
    const int row4 = world * w4;
    for (int i = c * blockDim.x + threadIdx.x; i < total; i += cpp * blockDim.x) {
        const int r = i / w4;
        const int j = i - r * w4;
        dst[static_cast<int64_t>(r) * row4 + rank * w4 + j] = local[i];
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();                       // the CTA's stores, ordered before the signal
        pg_signal(flag_table[peer] + rank);
        if (c == 0) {
            const uint32_t* mine = flag_table[rank] + peer;
            const unsigned long long t0 = pg_now_ns();
            bool ok = false;
            for (;;) {
                if (static_cast<int32_t>(pg_peek(mine) - target) >= 0) { ok = true; break; }
                if (pg_now_ns() - t0 > timeout_ns) break;
                __nanosleep(40);
            }
            if (!ok) atomicCAS(&state[2], 0u, static_cast<uint32_t>(1 + peer));
        }
        __threadfence();
        const uint32_t t = atomicAdd(&state[1], 1u);
        if (t == gridDim.x - 1) {                     // every CTA of this launch has read state[0]
            state[1] = 0;
            state[0] = target;
        }
    }
}

// The waiting half alone, for producers that push their results themselves (the sharded GEMM): thread p
// waits until rank p's counter here has grown by `add` over state[0], then state[0] advances.
__global__ void __launch_bounds__(64)
peer_wait_kernel(uint32_t* const* __restrict__ flag_table, uint32_t* __restrict__ state, int rank, int world,
                 uint32_t add, unsigned long long timeout_ns) {
    const uint32_t target = state[0] + add;
    if (static_cast<int>(threadIdx.x) < world) {
        const uint32_t* mine = flag_table[rank] + threadIdx.x;
        const unsigned long long t0 = pg_now_ns();
        bool ok = false;
        for (;;) {
            if (static_cast<int32_t>(pg_peek(mine) - target) >= 0) { ok = true; break; }
            if (pg_now_ns() - t0 > timeout_ns) break;
            __nanosleep(40);
        }
        if (!ok) atomicCAS(&state[2], 0u, static_cast<uint32_t>(1 + threadIdx.x));
    }
    __syncthreads();
    if (threadIdx.x == 0) state[0] = target;
}

int launch_peer_wait(uint32_t* const* flag_table, uint32_t* state, int rank, int world, uint32_t add,
                     int timeout_ms, cudaStream_t st) {
    if (!flag_table || !state) return LHB_ERR_NULL;
    if (world < 1 || world > 64 || rank < 0 || rank >= world || timeout_ms <= 0) return LHB_ERR_BAD_SHAPE;
    peer_wait_kernel<<<1, 64, 0, st>>>(flag_table, state, rank, world, add,
                                       static_cast<unsigned long long>(timeout_ms) * 1000000ull);
    LHB_LAUNCH_CHECK();
    return LHB_OK;
}

inline int peer_ctas_per_peer(int rows, int width) {
    const int64_t bytes = static_cast<int64_t>(rows) * width * 4;
    int cpp = static_cast<int>((bytes + 32767) / 32768);
    return cpp < 1 ? 1 : (cpp > 8 ? 8 : cpp);
}

}  // namespace lhb

using namespace lhb;

#define REQUIRE(cond, code) \
    do {                    \
        if (!(cond)) return (code); \
    } while (0)

extern "C" {

int lhb_peer_alloc(void** out, size_t bytes) {
    REQUIRE(out, LHB_ERR_NULL);
    REQUIRE(bytes > 0, LHB_ERR_BAD_SHAPE);
    void* p = nullptr;
    LHB_CUDA(cudaMalloc(&p, bytes));
    cudaError_t e = cudaMemset(p, 0, bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        set_last_error("cudaMemset(peer buffer)", e);
        cudaFree(p);
        return LHB_ERR_CUDA;
    }
    *out = p;
    return LHB_OK;
}

int lhb_peer_free(void* ptr) {
    if (!ptr) return LHB_OK;
    LHB_CUDA(cudaFree(ptr));
    return LHB_OK;
}

int lhb_peer_export(void* ptr, unsigned char* handle64) {
    REQUIRE(ptr && handle64, LHB_ERR_NULL);
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    cudaIpcMemHandle_t h;
    LHB_CUDA(cudaIpcGetMemHandle(&h, ptr));
    memcpy(handle64, &h, 64);
    return LHB_OK;
}

int lhb_peer_open(const unsigned char* handle64, void** out) {
    REQUIRE(handle64 && out, LHB_ERR_NULL);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    void* p = nullptr;
    LHB_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *out = p;
    return LHB_OK;
}

int lhb_peer_close(void* mapped) {
    if (!mapped) return LHB_OK;
    LHB_CUDA(cudaIpcCloseMemHandle(mapped));
    return LHB_OK;
}

int lhb_peer_allgather_cols(const float* local, int rows, int width, void* const* dst_table,
                            uint32_t* const* flag_table, uint32_t* state, int rank, int world, int timeout_ms,
                            void* stream) {
    REQUIRE(local && dst_table && flag_table && state, LHB_ERR_NULL);
    REQUIRE(rows >= 0 && width > 0 && (width & 3) == 0, LHB_ERR_BAD_SHAPE);
    REQUIRE(world >= 1 && world <= 64 && rank >= 0 && rank < world && timeout_ms > 0, LHB_ERR_BAD_SHAPE);
    REQUIRE(static_cast<int64_t>(rows) * width * world < (1ll << 31), LHB_ERR_BAD_SHAPE);
    REQUIRE(aligned16(local), LHB_ERR_MISALIGNED);
    if (rows == 0) return LHB_OK;
    const int cpp = peer_ctas_per_peer(rows, width);
    peer_allgather_cols_kernel<<<world * cpp, 512, 0, as_stream(stream)>>>(
        reinterpret_cast<const float4*>(local), rows, width / 4, reinterpret_cast<float4* const*>(dst_table),
        flag_table, state, rank, world, cpp, static_cast<unsigned long long>(timeout_ms) * 1000000ull);
    LHB_LAUNCH_CHECK();
    return LHB_OK;
}

int lhb_peer_status(const uint32_t* state, void* stream) {
    REQUIRE(state, LHB_ERR_NULL);
    uint32_t host[4] = {0, 0, 0, 0};
    LHB_CUDA(cudaMemcpyAsync(host, state, sizeof(host), cudaMemcpyDeviceToHost, as_stream(stream)));
    LHB_CUDA(cudaStreamSynchronize(as_stream(stream)));
    if (host[2] != 0) {
        set_last_error_text("peer all-gather: no arrival from rank " + std::to_string(host[2] - 1) +
                            " within the wait limit");
        return LHB_ERR_TIMEOUT;
    }
    return LHB_OK;
}

}  // extern "C"

// Device-resident cache manager.
//
// Host bookkeeping follows lh::CacheManager (src/runtime/cache_manager.cpp:8-102):
// a LIFO free list seeded so that pops ascend, per-block refcounts, recycled
// request ids and all-or-nothing ensure_capacity.  What moves to the GPU is the
// storage: int8 K/V pools with fp32 scale pools, and the batched block tables
// and seq_lens that lh::Scheduler::prepare_step rebuilds on the host every
// step (src/runtime/scheduler.cpp:41-58).  Here row `id` of a fixed
// [max_requests, max_blocks_per_req] table is patched in place when a request
// grows, so a decode step costs one 4-byte write per request (the seq_len bump)
// and one more every block_size steps.
#include <vector>

#include "common.cuh"

struct lhb_cache_manager {
    lhb_ctx* ctx = nullptr;
    lhb_paged_layout L{};
    int max_requests = 0;
    int max_blocks = 0;
    std::vector<int32_t> free_list;
    std::vector<int> refcount;
    std::vector<std::vector<int32_t>> tables;   // per request id
    std::vector<int> seq_len;
    std::vector<char> live;
    std::vector<int> recycled;
    int next_id = 0;
    int8_t* k_pool = nullptr;
    int8_t* v_pool = nullptr;
    float* k_scales = nullptr;
    float* v_scales = nullptr;
    int32_t* d_tables = nullptr;
    int32_t* d_seq_lens = nullptr;
};

using namespace lhb;

namespace {

__global__ void fill_i32_kernel(int32_t* p, int64_t n, int32_t v) {
    const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (i < n) p[i] = v;
}

int push_row(lhb_cache_manager* cm, int id, int from, int to, cudaStream_t st) {
    if (to <= from || !cm->d_tables) return LHB_OK;   // detached manager: host bookkeeping only
    LHB_CUDA(cudaMemcpyAsync(cm->d_tables + static_cast<int64_t>(id) * cm->max_blocks + from,
                             cm->tables[id].data() + from, sizeof(int32_t) * (to - from),
                             cudaMemcpyHostToDevice, st));
    return LHB_OK;
}

int take_block(lhb_cache_manager* cm) {
    if (cm->free_list.empty()) return -1;
    const int b = cm->free_list.back();
    cm->free_list.pop_back();
    cm->refcount[b] = 1;
    return b;
}

void drop_block(lhb_cache_manager* cm, int b) {
    if (b < 0 || b >= cm->L.num_blocks) return;
    int& rc = cm->refcount[b];
    if (rc <= 0) return;
    if (--rc == 0) cm->free_list.push_back(b);
}

bool valid_id(const lhb_cache_manager* cm, int id) {
    return cm && id >= 0 && id < cm->max_requests && cm->live[id];
}

}  // namespace

extern "C" {

int lhb_cm_create(lhb_ctx* ctx, const lhb_paged_layout* layout, int max_requests,
                  int max_blocks_per_req, lhb_cache_manager** out) {
    if (!layout || !out) return LHB_ERR_NULL;
    *out = nullptr;
    if (layout->num_blocks <= 0 || layout->block_size <= 0 || layout->n_kv_heads <= 0 ||
        layout->head_dim <= 0 || max_requests <= 0 || max_blocks_per_req <= 0)
        return LHB_ERR_BAD_SHAPE;
    if (ctx) LHB_CUDA(cudaSetDevice(ctx->device));
    auto* cm = new lhb_cache_manager();
    cm->ctx = ctx;
    cm->L = *layout;
    cm->max_requests = max_requests;
    cm->max_blocks = max_blocks_per_req;
    cm->refcount.assign(layout->num_blocks, 0);
    cm->free_list.reserve(layout->num_blocks);
    for (int i = layout->num_blocks - 1; i >= 0; --i) cm->free_list.push_back(i);
    cm->tables.resize(max_requests);
    cm->seq_len.assign(max_requests, 0);
    cm->live.assign(max_requests, 0);
    if (!ctx) { *out = cm; return LHB_OK; }   // detached: no device storage (host-side tests, planning)
    const size_t rows = static_cast<size_t>(layout->num_blocks) * layout->n_kv_heads * layout->block_size;
    const size_t pool = rows * layout->head_dim;
    const size_t tbl = static_cast<size_t>(max_requests) * max_blocks_per_req;
    bool ok = cudaMalloc(&cm->k_pool, pool) == cudaSuccess && cudaMalloc(&cm->v_pool, pool) == cudaSuccess &&
              cudaMalloc(&cm->k_scales, rows * 4) == cudaSuccess &&
              cudaMalloc(&cm->v_scales, rows * 4) == cudaSuccess &&
              cudaMalloc(&cm->d_tables, tbl * 4) == cudaSuccess &&
              cudaMalloc(&cm->d_seq_lens, static_cast<size_t>(max_requests) * 4) == cudaSuccess;
    if (!ok) {
        set_last_error("cudaMalloc(cache manager)", cudaGetLastError());
        lhb_cm_destroy(cm);
        return LHB_ERR_CUDA;
    }
    // the reference zero-fills its pools (src/runtime/cache_manager.cpp:12-13)
    cudaMemset(cm->k_pool, 0, pool);
    cudaMemset(cm->v_pool, 0, pool);
    cudaMemset(cm->k_scales, 0, rows * 4);
    cudaMemset(cm->v_scales, 0, rows * 4);
    cudaMemset(cm->d_seq_lens, 0, static_cast<size_t>(max_requests) * 4);
    fill_i32_kernel<<<static_cast<unsigned>((tbl + 255) / 256), 256>>>(cm->d_tables, tbl, -1);
    cudaDeviceSynchronize();
    *out = cm;
    return LHB_OK;
}

int lhb_cm_destroy(lhb_cache_manager* cm) {
    if (!cm) return LHB_ERR_NULL;
    if (cm->ctx) cudaSetDevice(cm->ctx->device);
    cudaFree(cm->k_pool); cudaFree(cm->v_pool); cudaFree(cm->k_scales); cudaFree(cm->v_scales);
    cudaFree(cm->d_tables); cudaFree(cm->d_seq_lens);
    delete cm;
    return LHB_OK;
}

int lhb_cm_num_free_blocks(const lhb_cache_manager* cm) { return cm ? static_cast<int>(cm->free_list.size()) : 0; }
int lhb_cm_num_total_blocks(const lhb_cache_manager* cm) { return cm ? cm->L.num_blocks : 0; }

int lhb_cm_create_request(lhb_cache_manager* cm) {
    if (!cm) return -1;
    int id;
    if (!cm->recycled.empty()) { id = cm->recycled.back(); cm->recycled.pop_back(); }
    else if (cm->next_id < cm->max_requests) id = cm->next_id++;
    else return -1;
    cm->live[id] = 1;
    cm->tables[id].clear();
    cm->seq_len[id] = 0;
    return id;
}

int lhb_cm_release_request(lhb_cache_manager* cm, int id, void* stream) {
    if (!cm) return LHB_ERR_NULL;
    if (!valid_id(cm, id)) return LHB_OK;              // reference: unknown id is a no-op
    cudaStream_t st = as_stream(stream);
    const int n = static_cast<int>(cm->tables[id].size());
    for (int32_t b : cm->tables[id]) drop_block(cm, b);
    cm->tables[id].assign(n, -1);
    const int e = push_row(cm, id, 0, n, st);
    cm->tables[id].clear();
    cm->seq_len[id] = 0;
    cm->live[id] = 0;
    cm->recycled.push_back(id);
    if (e) return e;
    if (cm->d_seq_lens) LHB_CUDA(cudaMemsetAsync(cm->d_seq_lens + id, 0, 4, st));
    return LHB_OK;
}

int lhb_cm_ensure_capacity(lhb_cache_manager* cm, int id, int seq_len, void* stream) {
    if (!cm) return LHB_ERR_NULL;
    if (!valid_id(cm, id) || seq_len < 0) return LHB_ERR_BAD_SHAPE;
    auto& t = cm->tables[id];
    const int needed = ceil_div(seq_len, cm->L.block_size);
    const int have = static_cast<int>(t.size());
    if (needed <= have) return 1;
    if (needed > cm->max_blocks) return 0;
    if (needed - have > static_cast<int>(cm->free_list.size())) return 0;   // no partial allocation
    for (int i = have; i < needed; ++i) t.push_back(take_block(cm));
    const int e = push_row(cm, id, have, needed, as_stream(stream));
    return e ? e : 1;
}

int lhb_cm_set_seq_len(lhb_cache_manager* cm, int id, int seq_len, void* stream) {
    if (!cm) return LHB_ERR_NULL;
    if (!valid_id(cm, id) || seq_len < 0) return LHB_ERR_BAD_SHAPE;
    cm->seq_len[id] = seq_len;
    if (cm->d_seq_lens) LHB_CUDA(cudaMemcpyAsync(cm->d_seq_lens + id, &cm->seq_len[id], 4, cudaMemcpyHostToDevice,
                             as_stream(stream)));
    return LHB_OK;
}

int lhb_cm_reference_block(lhb_cache_manager* cm, int id, int logical_idx, int physical,
                           void* stream) {
    if (!cm) return LHB_ERR_NULL;
    if (!valid_id(cm, id)) return LHB_ERR_BAD_SHAPE;
    if (logical_idx < 0 || logical_idx >= cm->max_blocks) return 0;
    auto& t = cm->tables[id];
    const int have = static_cast<int>(t.size());
    if (logical_idx < have) {
        if (t[logical_idx] >= 0) drop_block(cm, t[logical_idx]);
    } else {
        t.resize(logical_idx + 1, -1);
    }
    if (physical >= 0 && physical < cm->L.num_blocks) ++cm->refcount[physical];
    t[logical_idx] = physical;
    const int e = push_row(cm, id, std::min(have, logical_idx), logical_idx + 1, as_stream(stream));
    return e ? e : 1;
}

int lhb_cm_allocate_block(lhb_cache_manager* cm) { return cm ? take_block(cm) : -1; }
int lhb_cm_release_block(lhb_cache_manager* cm, int b) { if (!cm) return LHB_ERR_NULL; drop_block(cm, b); return LHB_OK; }
int lhb_cm_retain_block(lhb_cache_manager* cm, int b) {
    if (!cm) return LHB_ERR_NULL;
    if (b >= 0 && b < cm->L.num_blocks) ++cm->refcount[b];
    return LHB_OK;
}
int lhb_cm_refcount(const lhb_cache_manager* cm, int b) {
    return (cm && b >= 0 && b < cm->L.num_blocks) ? cm->refcount[b] : 0;
}
int lhb_cm_seq_len(const lhb_cache_manager* cm, int id) { return valid_id(cm, id) ? cm->seq_len[id] : 0; }
int lhb_cm_block_table(const lhb_cache_manager* cm, int id, int32_t* out, int cap) {
    if (!valid_id(cm, id)) return 0;
    const auto& t = cm->tables[id];
    for (int i = 0; i < static_cast<int>(t.size()) && i < cap; ++i) out[i] = t[i];
    return static_cast<int>(t.size());
}
int8_t* lhb_cm_k_pool(lhb_cache_manager* cm) { return cm ? cm->k_pool : nullptr; }
int8_t* lhb_cm_v_pool(lhb_cache_manager* cm) { return cm ? cm->v_pool : nullptr; }
float* lhb_cm_k_scales(lhb_cache_manager* cm) { return cm ? cm->k_scales : nullptr; }
float* lhb_cm_v_scales(lhb_cache_manager* cm) { return cm ? cm->v_scales : nullptr; }
int32_t* lhb_cm_block_tables(lhb_cache_manager* cm) { return cm ? cm->d_tables : nullptr; }
int32_t* lhb_cm_seq_lens(lhb_cache_manager* cm) { return cm ? cm->d_seq_lens : nullptr; }
int lhb_cm_max_blocks_per_req(const lhb_cache_manager* cm) { return cm ? cm->max_blocks : 0; }

}  // extern "C"

// ---------------------------------------------------------------------------
// Continuous-batching scheduler over the device cache manager.
//
// Lifecycle rules are lh::Scheduler's (src/runtime/scheduler.cpp:11-102): FIFO
// admission gated by the active-set cap and by all-or-nothing reservation of
// prompt + 1 tokens, no admission past a blocked queue head; every committed
// step counts one produced token, retires a request on its flag or on
// max_new_tokens, otherwise reserves the next slot (retiring the request if the
// pool is exhausted) and bumps its length.
//
// What differs is where the step view lives.  The reference rebuilds a dense
// [n_active, max_blocks] table on the host every step (scheduler.cpp:41-58).
// Here the per-request rows already sit in device memory (patched in place by
// the cache manager), so prepare_step uploads only the active request ids
// (4 bytes each) and a gather kernel writes the dense table and seq_lens of the
// active set, in active order, into device buffers the batched kernels read.
// Its width is the table's fixed max_blocks_per_req, not the step's maximum.
// ---------------------------------------------------------------------------
#include <deque>
#include <unordered_map>

struct lhb_scheduler {
    lhb_cache_manager* cm = nullptr;
    int max_concurrent = 0;
    struct Req { int prompt_len; int max_new; };
    std::deque<std::pair<int, Req>> queue;
    struct Active { Req req; int produced; };
    std::unordered_map<int, Active> active;
    std::vector<int> order;                       // active ids in prepare_step order
    std::unordered_map<int, int> generated;
    double last_occ = 0.0;
    int32_t* d_ids = nullptr;                     // [max_concurrent]
    int32_t* d_tables = nullptr;                  // [max_concurrent, max_blocks]
    int32_t* d_seq_lens = nullptr;                // [max_concurrent]
    int32_t* h_ids = nullptr;                     // pinned staging for the id upload
};

namespace {

__global__ void gather_active_kernel(const int32_t* __restrict__ ids, const int32_t* __restrict__ all_tables,
                                     const int32_t* __restrict__ all_lens, int32_t* __restrict__ tables,
                                     int32_t* __restrict__ lens, int max_blocks) {
    const int row = blockIdx.x, id = ids[row];
    for (int b = threadIdx.x; b < max_blocks; b += blockDim.x)
        tables[static_cast<int64_t>(row) * max_blocks + b] = all_tables[static_cast<int64_t>(id) * max_blocks + b];
    if (threadIdx.x == 0) lens[row] = all_lens[id];
}

bool sched_try_admit(lhb_scheduler* s, int id, const lhb_scheduler::Req& r, void* stream) {
    if (lhb_cm_ensure_capacity(s->cm, id, r.prompt_len + 1, stream) != 1) return false;
    lhb_cm_set_seq_len(s->cm, id, r.prompt_len, stream);
    s->active.emplace(id, lhb_scheduler::Active{r, 0});
    s->order.push_back(id);
    return true;
}

void sched_retire(lhb_scheduler* s, int id, int produced, void* stream) {
    s->generated[id] = produced;
    lhb_cm_release_request(s->cm, id, stream);
    s->active.erase(id);
}

}  // namespace

extern "C" {

int lhb_sched_create(lhb_cache_manager* cm, int max_concurrent, lhb_scheduler** out) {
    if (!cm || !out) return LHB_ERR_NULL;
    if (max_concurrent < 0 || max_concurrent > cm->max_requests) return LHB_ERR_BAD_SHAPE;
    auto* s = new lhb_scheduler();
    s->cm = cm;
    s->max_concurrent = max_concurrent;
    if (cm->ctx && max_concurrent > 0) {
        const size_t n = static_cast<size_t>(max_concurrent);
        if (cudaMalloc(&s->d_ids, n * 4) != cudaSuccess || cudaMalloc(&s->d_seq_lens, n * 4) != cudaSuccess ||
            cudaMalloc(&s->d_tables, n * cm->max_blocks * 4) != cudaSuccess ||
            cudaMallocHost(&s->h_ids, n * 4) != cudaSuccess) {
            cudaGetLastError();
            lhb_sched_destroy(s);
            return LHB_ERR_CUDA;
        }
    }
    *out = s;
    return LHB_OK;
}

int lhb_sched_destroy(lhb_scheduler* s) {
    if (!s) return LHB_OK;
    cudaFree(s->d_ids);
    cudaFree(s->d_seq_lens);
    cudaFree(s->d_tables);
    cudaFreeHost(s->h_ids);
    delete s;
    return LHB_OK;
}

int lhb_sched_submit(lhb_scheduler* s, int prompt_len, int max_new_tokens) {
    if (!s || prompt_len < 0) return -1;
    const int id = lhb_cm_create_request(s->cm);
    if (id < 0) return -1;
    s->queue.emplace_back(id, lhb_scheduler::Req{prompt_len, max_new_tokens});
    return id;
}

int lhb_sched_has_work(const lhb_scheduler* s) { return s && (!s->queue.empty() || !s->active.empty()) ? 1 : 0; }
int lhb_sched_queue_depth(const lhb_scheduler* s) { return s ? static_cast<int>(s->queue.size()) : 0; }
int lhb_sched_active_size(const lhb_scheduler* s) { return s ? static_cast<int>(s->active.size()) : 0; }
double lhb_sched_last_step_occupancy(const lhb_scheduler* s) { return s ? s->last_occ : 0.0; }
int lhb_sched_generated(const lhb_scheduler* s, int id) {
    if (!s) return 0;
    auto it = s->generated.find(id);
    return it == s->generated.end() ? 0 : it->second;
}

int lhb_sched_prepare_step(lhb_scheduler* s, int32_t* ids_out, int cap, void* stream) {
    if (!s) return LHB_ERR_NULL;
    while (!s->queue.empty() && static_cast<int>(s->active.size()) < s->max_concurrent) {
        auto& head = s->queue.front();
        if (!sched_try_admit(s, head.first, head.second, stream)) break;
        s->queue.pop_front();
    }
    const int n = static_cast<int>(s->order.size());
    s->last_occ = s->max_concurrent > 0 ? static_cast<double>(s->active.size()) / s->max_concurrent : 0.0;
    if (ids_out) {
        if (cap < n) return LHB_ERR_BAD_SHAPE;
        for (int i = 0; i < n; ++i) ids_out[i] = s->order[i];
    }
    if (s->cm->ctx && n > 0) {
        cudaStream_t st = as_stream(stream);
        // the staging buffer may still be in flight from the previous step on another stream
        LHB_CUDA(cudaStreamSynchronize(st));
        for (int i = 0; i < n; ++i) s->h_ids[i] = s->order[i];
        LHB_CUDA(cudaMemcpyAsync(s->d_ids, s->h_ids, sizeof(int32_t) * n, cudaMemcpyHostToDevice, st));
        gather_active_kernel<<<n, 128, 0, st>>>(s->d_ids, s->cm->d_tables, s->cm->d_seq_lens, s->d_tables,
                                                s->d_seq_lens, s->cm->max_blocks);
        LHB_LAUNCH_CHECK();
    }
    return n;
}

int lhb_sched_commit_step(lhb_scheduler* s, const uint8_t* completed, int n, void* stream) {
    if (!s || (!completed && n > 0)) return LHB_ERR_NULL;
    if (n != static_cast<int>(s->order.size())) return LHB_ERR_BAD_SHAPE;
    std::vector<int> survivors;
    survivors.reserve(s->order.size());
    for (int i = 0; i < n; ++i) {
        const int id = s->order[i];
        auto it = s->active.find(id);
        if (it == s->active.end()) continue;
        auto& st = it->second;
        ++st.produced;
        if (completed[i] || st.produced >= st.req.max_new) {
            sched_retire(s, id, st.produced, stream);
            continue;
        }
        const int new_len = lhb_cm_seq_len(s->cm, id) + 1;
        if (lhb_cm_ensure_capacity(s->cm, id, new_len + 1, stream) != 1) {   // pool exhausted: finish early
            sched_retire(s, id, st.produced, stream);
            continue;
        }
        lhb_cm_set_seq_len(s->cm, id, new_len, stream);
        survivors.push_back(id);
    }
    s->order.swap(survivors);
    return LHB_OK;
}

int32_t* lhb_sched_block_tables(lhb_scheduler* s) { return s ? s->d_tables : nullptr; }
int32_t* lhb_sched_seq_lens(lhb_scheduler* s) { return s ? s->d_seq_lens : nullptr; }
int lhb_sched_max_blocks_per_req(const lhb_scheduler* s) { return s ? s->cm->max_blocks : 0; }

}  // extern "C"

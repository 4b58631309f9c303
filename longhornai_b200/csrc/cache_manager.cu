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

// TMA tensor-map construction.  cuTensorMapEncodeTiled is resolved at run time
// through the CUDA runtime's driver entry-point query, so the library carries
// no link-time dependency on libcuda and still loads on a machine without a
// driver (where every compute call reports LHB_ERR_CUDA).
#include <cuda.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <string>

#include "common.cuh"
#include "dispatch.h"

namespace lhb {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn resolve_encode() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
        else
            cudaGetLastError();
    });
    return fn;
}

static_assert(sizeof(TensorMap) == sizeof(CUtensorMap), "tensor map blob size");

static int get_tensor_map_2d(lhb_ctx* ctx, CUtensorMapDataType dtype, const void* base, uint64_t rows,
                             uint64_t cols, uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols,
                             bool swizzle128, TensorMap* out) {
    char key[160];
    snprintf(key, sizeof(key), "%d/%p/%llu/%llu/%llu/%u/%u/%d", (int)dtype, base, (unsigned long long)rows,
             (unsigned long long)cols, (unsigned long long)pitch_bytes, box_rows, box_cols,
             swizzle128 ? 1 : 0);
    {
        std::lock_guard<std::mutex> lk(ctx->mu);
        auto it = ctx->tmaps.find(key);
        if (it != ctx->tmaps.end()) { *out = it->second; return LHB_OK; }
    }
    EncodeTiledFn enc = resolve_encode();
    if (!enc) { set_last_error_text("cuTensorMapEncodeTiled unavailable"); return LHB_ERR_CUDA; }
    if ((reinterpret_cast<uintptr_t>(base) & 15) || (pitch_bytes & 15)) return LHB_ERR_MISALIGNED;
    CUtensorMap tm;
    const cuuint64_t gdim[2] = {cols, rows};
    const cuuint64_t gstride[1] = {pitch_bytes};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(&tm, dtype, 2, const_cast<void*>(base), gdim,
                           gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_last_error_text("cuTensorMapEncodeTiled failed with CUresult " + std::to_string((int)r));
        return LHB_ERR_CUDA;
    }
    memcpy(out->bytes, &tm, sizeof(tm));
    std::lock_guard<std::mutex> lk(ctx->mu);
    if (ctx->tmaps.size() > 4096) ctx->tmaps.clear();
    ctx->tmaps[key] = *out;
    return LHB_OK;
}

int get_tensor_map_2d_u8(lhb_ctx* ctx, const void* base, uint64_t rows, uint64_t cols,
                         uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols,
                         bool swizzle128, TensorMap* out) {
    return get_tensor_map_2d(ctx, CU_TENSOR_MAP_DATA_TYPE_UINT8, base, rows, cols, pitch_bytes, box_rows,
                             box_cols, swizzle128, out);
}

int get_tensor_map_2d_f32(lhb_ctx* ctx, const void* base, uint64_t rows, uint64_t cols,
                          uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols, TensorMap* out) {
    return get_tensor_map_2d(ctx, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, base, rows, cols, pitch_bytes, box_rows,
                             box_cols, false, out);
}

int get_tensor_map_2d_f32_sw128(lhb_ctx* ctx, const void* base, uint64_t rows, uint64_t cols,
                                uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols, TensorMap* out) {
    return get_tensor_map_2d(ctx, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, base, rows, cols, pitch_bytes, box_rows,
                             box_cols, true, out);
}

int get_tensor_map_2d_f16(lhb_ctx* ctx, const void* base, uint64_t rows, uint64_t cols,
                          uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols, TensorMap* out) {
    return get_tensor_map_2d(ctx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, base, rows, cols, pitch_bytes, box_rows,
                             box_cols, false, out);
}

}  // namespace lhb

namespace lhb {
const Knobs& knobs() {
    static const Knobs k = [] {
        Knobs v;
        auto num = [](const char* name, int unset) {
            const char* e = getenv(name);
            return e ? atoi(e) : unset;
        };
        v.pdl = num("LHB_PDL", 1) != 0;
        v.w4tc_min_m = std::max(1, num("LHB_W4TC_MIN_M", 9));
        v.w4tc_stream_k = num("LHB_W4TC_SPLIT", 0) == 1;
        v.w4tc_ctas = std::max(0, num("LHB_W4TC_CTAS", 0));
        v.w4tc_coop = num("LHB_W4TC_COOP", 1) != 0;
        v.w8a8_pair = num("LHB_W8A8_PAIR", 1) != 0;
        const char* push = getenv("LHB_W8A8_PUSH");
        v.w8a8_push_tma = !(push && push[0] == 's');
        v.gemv_ctas_per_sm = std::max(0, num("LHB_GEMV_CTAS_PER_SM", 0));
        v.gemv_smem_kb = std::max(0, num("LHB_GEMV_SMEM_KB", 0));
        v.decode_target = std::max(0, num("LHB_DECODE_TARGET", 0));
        v.decode_pages = std::max(0, num("LHB_DECODE_PAGES", 0));
        v.decode_splits = std::max(0, num("LHB_DECODE_SPLITS", 0));
        v.decode_one_wave = num("LHB_DECODE_ONE_WAVE", 1) != 0;
        return v;
    }();
    return k;
}
}  // namespace lhb

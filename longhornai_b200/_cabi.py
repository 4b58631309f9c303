"""ctypes binding of liblhb200.so (the C ABI declared in include/lhb200.h).

The library is the product; this module only loads it and declares argument
types.  If the shared object is missing it is built with nvcc; if it cannot be
loaded, importing fails loudly -- there is no fallback implementation.
"""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "lib", "liblhb200.so")

OK = 0
ERR_BAD_SHAPE, ERR_MISALIGNED, ERR_UNSUPPORTED, ERR_CUDA, ERR_NULL, ERR_SCRATCH, ERR_TIMEOUT = (
    -1, -2, -3, -4, -5, -6, -7)


class PagedLayout(C.Structure):
    """lhb_paged_layout == lh::PagedCacheLayout (src/kernels/kvcache.hpp:26-31)."""
    _fields_ = [("num_blocks", C.c_int), ("block_size", C.c_int),
                ("n_kv_heads", C.c_int), ("head_dim", C.c_int)]


class PagedAttnCfg(C.Structure):
    """lhb_paged_attn_cfg == lh::PagedAttnConfig (src/kernels/paged_attention.hpp:28-37)."""
    _fields_ = [("n_q_heads", C.c_int), ("n_kv_heads", C.c_int), ("seq_q", C.c_int),
                ("head_dim", C.c_int), ("causal", C.c_int), ("scale", C.c_float),
                ("window", C.c_int), ("chunk", C.c_int)]


_vp, _i, _f, _sz = C.c_void_p, C.c_int, C.c_float, C.c_size_t
_LP, _CP = C.POINTER(PagedLayout), C.POINTER(PagedAttnCfg)

# name -> (restype, argtypes); mirrors include/lhb200.h one to one
SIGNATURES = {
    "lhb_ctx_create": (_i, [_i, _sz, C.POINTER(_vp)]),
    "lhb_ctx_destroy": (_i, [_vp]),
    "lhb_ctx_poll": (_i, [_vp, _vp]),
    "lhb_ctx_set_sm_limit": (_i, [_vp, _i]),
    "lhb_gemm_w8a8_sharded": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _vp]),
    "lhb_status_string": (C.c_char_p, [_i]),
    "lhb_last_error": (C.c_char_p, []),
    "lhb_gemm_w4a16_fast_path": (_i, [_i, _i, _i, _i]),
    "lhb_gemm_w8a16_fast_path": (_i, [_i, _i, _i]),
    "lhb_gemm_w8a8_fast_path": (_i, [_i, _i, _i]),
    "lhb_paged_attention_q8_fast_path": (_i, [_CP, _LP]),
    "lhb_q8_quantize_per_tensor": (_i, [_vp, _vp, _vp, _vp, C.c_int64, _vp]),
    "lhb_q8_dequantize_per_tensor": (_i, [_vp, _vp, _f, _vp, C.c_int64, _vp]),
    "lhb_q8_quantize_per_row": (_i, [_vp, _vp, _vp, _vp, _i, _i, _vp]),
    "lhb_q8_dequantize_per_row": (_i, [_vp, _vp, _vp, _vp, _i, _i, _vp]),
    "lhb_q8_quantize_per_col": (_i, [_vp, _vp, _vp, _vp, _i, _i, _vp]),
    "lhb_q8_dequantize_per_col": (_i, [_vp, _vp, _vp, _vp, _i, _i, _vp]),
    "lhb_q4_quantize_groupwise": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "lhb_q4_dequantize_groupwise": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "lhb_rmsnorm": (_i, [_vp, _vp, _vp, _vp, _i, _i, _f, _vp]),
    "lhb_rope": (_i, [_vp, _vp, _i, _i, _i, _f, _f, _i, _i, _vp]),
    "lhb_rope_decode_batched": (_i, [_vp, _vp, _vp, _i, _i, _i, _f, _f, _i, _vp]),
    "lhb_swiglu": (_i, [_vp, _vp, _vp, _i, _i, _vp]),
    "lhb_gemm_w4a16_groupwise_prologue": (_i, [_vp, _vp, _i, _vp, _f, _vp, _vp, _vp, _i, _i, _i, _i, _f, _f, _vp]),
    "lhb_qkv_rope_append_q8_decode": (_i, [_vp, _vp, C.c_int64, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _i, _i, _LP,
                                           _f, _f, _i, _vp]),
    "lhb_fp8_quantize_per_tensor": (_i, [_vp, _vp, _vp, _vp, C.c_int64, _vp]),
    "lhb_fp8_quantize_per_row": (_i, [_vp, _vp, _vp, _vp, _i, _i, _vp]),
    "lhb_fp8_quantize_per_col": (_i, [_vp, _vp, _vp, _vp, _i, _i, _vp]),
    "lhb_fp8_dequantize": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "lhb_gemm_fp8_e4m3": (_i, [_vp, _vp, _vp, _f, _f, _vp, _i, _i, _i, _f, _f, _vp]),
    "lhb_gemm_fp8_fast_path": (_i, [_i, _i, _i]),
    "lhb_q4a_quantize_groupwise": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "lhb_q4a_dequantize_groupwise": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "lhb_gemm_w4a16_asym": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _f, _vp]),
    "lhb_gemm_w4a16_asym_fast_path": (_i, [_i, _i, _i, _i]),
    "lhb_gemm_w8a8": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _f, _f, _vp]),
    "lhb_gemm_w4a16_groupwise": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _f, _vp]),
    "lhb_gemm_w8a16_perchannel": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _f, _f, _vp]),
    "lhb_paged_kv_append_q8": (_i, [_vp] * 8 + [_LP, _i, _i, _vp]),
    "lhb_paged_kv_append_q8_batched": (_i, [_vp] * 8 + [_i, _vp, _i, _LP, _i, _vp]),
    "lhb_paged_kv_append_f32": (_i, [_vp] * 6 + [_LP, _i, _i, _vp]),
    "lhb_paged_attention_q8": (_i, [_vp] * 7 + [_i, _vp, _CP, _LP, _vp]),
    "lhb_paged_attention_q8_batched": (_i, [_vp] * 7 + [_i, _vp, _i, _vp, _CP, _LP, _vp]),
    "lhb_paged_attention_q8_batched_noalloc": (_i, [_vp] * 6 + [_i, _vp, _i, _vp, _CP, _LP, _vp]),
    "lhb_paged_attention_f32_batched": (_i, [_vp] * 5 + [_i, _vp, _i, _vp, _CP, _LP, _vp]),
    "lhb_cm_create": (_i, [_vp, _LP, _i, _i, C.POINTER(_vp)]),
    "lhb_cm_destroy": (_i, [_vp]),
    "lhb_cm_num_free_blocks": (_i, [_vp]),
    "lhb_cm_num_total_blocks": (_i, [_vp]),
    "lhb_cm_create_request": (_i, [_vp]),
    "lhb_cm_release_request": (_i, [_vp, _i, _vp]),
    "lhb_cm_ensure_capacity": (_i, [_vp, _i, _i, _vp]),
    "lhb_cm_set_seq_len": (_i, [_vp, _i, _i, _vp]),
    "lhb_cm_reference_block": (_i, [_vp, _i, _i, _i, _vp]),
    "lhb_cm_allocate_block": (_i, [_vp]),
    "lhb_cm_release_block": (_i, [_vp, _i]),
    "lhb_cm_retain_block": (_i, [_vp, _i]),
    "lhb_cm_refcount": (_i, [_vp, _i]),
    "lhb_cm_seq_len": (_i, [_vp, _i]),
    "lhb_cm_block_table": (_i, [_vp, _i, _vp, _i]),
    "lhb_cm_k_pool": (_vp, [_vp]),
    "lhb_cm_v_pool": (_vp, [_vp]),
    "lhb_cm_k_scales": (_vp, [_vp]),
    "lhb_cm_v_scales": (_vp, [_vp]),
    "lhb_cm_block_tables": (_vp, [_vp]),
    "lhb_cm_seq_lens": (_vp, [_vp]),
    "lhb_cm_max_blocks_per_req": (_i, [_vp]),
    "lhb_sched_create": (_i, [_vp, _i, C.POINTER(_vp)]),
    "lhb_sched_destroy": (_i, [_vp]),
    "lhb_sched_submit": (_i, [_vp, _i, _i]),
    "lhb_sched_has_work": (_i, [_vp]),
    "lhb_sched_queue_depth": (_i, [_vp]),
    "lhb_sched_active_size": (_i, [_vp]),
    "lhb_sched_last_step_occupancy": (C.c_double, [_vp]),
    "lhb_sched_generated": (_i, [_vp, _i]),
    "lhb_sched_prepare_step": (_i, [_vp, _vp, _i, _vp]),
    "lhb_sched_commit_step": (_i, [_vp, _vp, _i, _vp]),
    "lhb_sched_block_tables": (_vp, [_vp]),
    "lhb_sched_seq_lens": (_vp, [_vp]),
    "lhb_sched_max_blocks_per_req": (_i, [_vp]),
    "lhb_peer_alloc": (_i, [C.POINTER(_vp), C.c_size_t]),
    "lhb_peer_free": (_i, [_vp]),
    "lhb_peer_alloc_shareable": (_i, [C.POINTER(_vp), C.c_size_t, C.POINTER(_i), C.POINTER(C.c_size_t)]),
    "lhb_peer_open_fd": (_i, [_i, C.c_size_t, C.POINTER(_vp)]),
    "lhb_peer_unmap": (_i, [_vp, C.c_size_t]),
    "lhb_peer_export": (_i, [_vp, _vp]),
    "lhb_peer_open": (_i, [_vp, C.POINTER(_vp)]),
    "lhb_peer_close": (_i, [_vp]),
    "lhb_peer_allgather_cols": (_i, [_vp, _i, _i, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "lhb_peer_status": (_i, [_vp, _vp]),
    "lhb_gemm_w4a16_groupwise_peer": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, C.c_float, C.c_float, _vp, _vp, _vp,
                                           _i, _i, _i, _vp]),
}

_lib = None


def load(build_if_missing: bool = True) -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        if not build_if_missing:
            raise ImportError(f"{LIB_PATH} is missing: run `python -m longhornai_b200.build`")
        from . import build as _build
        _build.build()
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError here = header/library mismatch
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


class LhbError(RuntimeError):
    def __init__(self, status: int, where: str):
        lib = load()
        msg = lib.lhb_status_string(status).decode()
        detail = lib.lhb_last_error().decode()
        super().__init__(f"{where}: {msg} ({status})" + (f": {detail}" if status == ERR_CUDA and detail else ""))
        self.status = status


def last_error() -> str:
    """Text of the last failed CUDA / driver call on this thread (empty when there was none)."""
    return load().lhb_last_error().decode()


def check(status: int, where: str) -> None:
    if status != OK:
        raise LhbError(status, where)

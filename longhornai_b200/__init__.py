"""longhornai_b200 -- B200 (sm_100a) implementation of LonghornAI's quantized
decode hot path: gemm_quant (W4A16 group-wise, weight-only int8, W8A8),
kvcache_quant (int8 paged KV append) and paged_attention decode.

The product is the C-ABI library ``lib/liblhb200.so`` (``include/lhb200.h``)
built from ``csrc/``.  This package is the thin host-side mirror of the
reference's ``namespace lh`` free functions over that ABI: same names, same
argument order and meaning, operating on CUDA tensors (PyTorch is used for
device memory and streams only).  There is no CPU or eager fallback.
"""
from . import _cabi
from ._cabi import LhbError, PagedAttnCfg, PagedLayout
from .kernels import (Context, default_context, gemm_w4a16_groupwise, gemm_w8a8,
                      gemm_w8a16_perchannel, paged_attention_batched_f32, paged_attention_q8,
                      paged_attention_q8_batched, paged_attention_q8_batched_noalloc, paged_kv_append, paged_kv_append_q8,
                      paged_kv_append_q8_batched, q4_dequantize_groupwise, q4_quantize_groupwise,
                      q8_dequantize_per_col, q8_dequantize_per_row, q8_quantize_per_col,
                      q8_dequantize_per_tensor, q8_quantize_per_tensor,
                      q8_quantize_per_row, rmsnorm, rope, rope_decode_batched, swiglu,
                      gemm_w4a16_asym, q4a_dequantize_groupwise, q4a_quantize_groupwise,
                      fp8_dequantize, fp8_quantize_per_col, fp8_quantize_per_row, fp8_quantize_per_tensor,
                      gemm_fp8_e4m3, qkv_rope_append_q8_decode, gemm_w4a16_norm, gemm_w4a16_swiglu)
from .runtime import ActiveStep, DeviceCacheManager, DeviceScheduler

__all__ = [n for n in dir() if not n.startswith("_")]

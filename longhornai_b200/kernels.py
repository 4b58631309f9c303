"""Host-side mirror of the reference's kernel functions over the C ABI.

Function names, argument order and semantics follow ``namespace lh``
(src/kernels/quant.hpp, gemm_quant.hpp, kvcache_quant.hpp,
paged_attention.hpp of the reference); tensors replace raw pointers and shapes
are read from them.  Every function enqueues on the current CUDA stream of the
tensor's device and returns without synchronising.  Inputs must be contiguous
CUDA tensors of the documented dtype; anything else raises (no silent copies,
no CPU path).
"""
from __future__ import annotations

import ctypes as C
import threading

import torch

from . import _cabi
from ._cabi import PagedAttnCfg, PagedLayout, check


class Context:
    """Per-device library context (scratch arena + status word)."""

    def __init__(self, device: int | None = None, scratch_bytes: int = 0):
        if not torch.cuda.is_available():
            raise RuntimeError("longhornai_b200 needs a CUDA device: there is no CPU fallback")
        self.device = torch.cuda.current_device() if device is None else int(device)
        self.lib = _cabi.load()
        h = C.c_void_p()
        with torch.cuda.device(self.device):
            check(self.lib.lhb_ctx_create(self.device, scratch_bytes, C.byref(h)), "lhb_ctx_create")
        self.handle = h

    def poll(self) -> int:
        """Synchronise the current stream and return (and clear) the device status word."""
        return int(self.lib.lhb_ctx_poll(self.handle, _stream(self.device)))

    def set_sm_limit(self, n: int) -> None:
        """The persistent tensor-core grids of this context use at most `n` SMs (0 = all), leaving the
        rest to kernels the caller runs beside them."""
        check(self.lib.lhb_ctx_set_sm_limit(self.handle, int(n)), "lhb_ctx_set_sm_limit")

    def close(self):
        if getattr(self, "handle", None):
            self.lib.lhb_ctx_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_ctx_lock = threading.Lock()
_contexts: dict[int, Context] = {}


def default_context(device: int | None = None) -> Context:
    dev = torch.cuda.current_device() if device is None else int(device)
    with _ctx_lock:
        if dev not in _contexts:
            _contexts[dev] = Context(dev)
        return _contexts[dev]


def _stream(device: int):
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _t(x: torch.Tensor, dtype, name: str) -> int:
    if not isinstance(x, torch.Tensor) or not x.is_cuda:
        raise TypeError(f"{name}: expected a CUDA tensor (no CPU path)")
    if x.dtype != dtype:
        raise TypeError(f"{name}: expected {dtype}, got {x.dtype}")
    if not x.is_contiguous():
        raise ValueError(f"{name}: must be contiguous")
    return x.data_ptr()


def _ctx_for(x: torch.Tensor, ctx: Context | None) -> Context:
    return ctx if ctx is not None else default_context(x.device.index)


# ---------------------------------------------------------------------------
# quantisers  (src/kernels/quant.hpp:38-63)
# ---------------------------------------------------------------------------

def q8_quantize_per_tensor(src: torch.Tensor, ctx: Context | None = None):
    """lh::q8_quantize_per_tensor (src/kernels/quant.hpp:31): fp32 tensor -> (int8 of the same shape,
    fp32 scale [1] on the device); bit-exact."""
    c = _ctx_for(src, ctx)
    dst = torch.empty(src.shape, dtype=torch.int8, device=src.device)
    scale = torch.empty(1, dtype=torch.float32, device=src.device)
    check(c.lib.lhb_q8_quantize_per_tensor(c.handle, _t(src, torch.float32, "src"), dst.data_ptr(),
                                           scale.data_ptr(), src.numel(), _stream(c.device)),
          "q8_quantize_per_tensor")
    return dst, scale


def q8_dequantize_per_tensor(src, scale: float, ctx=None):
    c = _ctx_for(src, ctx)
    dst = torch.empty(src.shape, dtype=torch.float32, device=src.device)
    check(c.lib.lhb_q8_dequantize_per_tensor(c.handle, _t(src, torch.int8, "src"), C.c_float(float(scale)),
                                             dst.data_ptr(), src.numel(), _stream(c.device)),
          "q8_dequantize_per_tensor")
    return dst


def q8_quantize_per_row(src: torch.Tensor, ctx: Context | None = None):
    """fp32 [rows, dim] -> (int8 [rows, dim], fp32 scales [rows]); bit-exact."""
    c = _ctx_for(src, ctx)
    rows, dim = src.shape
    dst = torch.empty((rows, dim), dtype=torch.int8, device=src.device)
    scales = torch.empty(rows, dtype=torch.float32, device=src.device)
    check(c.lib.lhb_q8_quantize_per_row(c.handle, _t(src, torch.float32, "src"), dst.data_ptr(),
                                        scales.data_ptr(), rows, dim, _stream(c.device)),
          "q8_quantize_per_row")
    return dst, scales


def q8_dequantize_per_row(src, scales, ctx=None):
    c = _ctx_for(src, ctx)
    rows, dim = src.shape
    dst = torch.empty((rows, dim), dtype=torch.float32, device=src.device)
    check(c.lib.lhb_q8_dequantize_per_row(c.handle, _t(src, torch.int8, "src"),
                                          _t(scales, torch.float32, "scales"), dst.data_ptr(), rows,
                                          dim, _stream(c.device)), "q8_dequantize_per_row")
    return dst


def q8_quantize_per_col(src, ctx=None):
    """fp32 [rows, cols] -> (int8 [rows, cols], fp32 scales [cols]); bit-exact."""
    c = _ctx_for(src, ctx)
    rows, cols = src.shape
    dst = torch.empty((rows, cols), dtype=torch.int8, device=src.device)
    scales = torch.empty(cols, dtype=torch.float32, device=src.device)
    check(c.lib.lhb_q8_quantize_per_col(c.handle, _t(src, torch.float32, "src"), dst.data_ptr(),
                                        scales.data_ptr(), rows, cols, _stream(c.device)),
          "q8_quantize_per_col")
    return dst, scales


def q8_dequantize_per_col(src, scales, ctx=None):
    c = _ctx_for(src, ctx)
    rows, cols = src.shape
    dst = torch.empty((rows, cols), dtype=torch.float32, device=src.device)
    check(c.lib.lhb_q8_dequantize_per_col(c.handle, _t(src, torch.int8, "src"),
                                          _t(scales, torch.float32, "scales"), dst.data_ptr(), rows,
                                          cols, _stream(c.device)), "q8_dequantize_per_col")
    return dst


def q4_quantize_groupwise(src, group_size: int, ctx=None):
    """fp32 [K, N] -> (uint8 packed [K/2, N], fp32 scales [K/G, N]); bit-exact."""
    c = _ctx_for(src, ctx)
    K, N = src.shape
    packed = torch.empty((K // 2, N), dtype=torch.uint8, device=src.device)
    scales = torch.empty((K // group_size, N), dtype=torch.float32, device=src.device)
    check(c.lib.lhb_q4_quantize_groupwise(c.handle, _t(src, torch.float32, "src"), packed.data_ptr(),
                                          scales.data_ptr(), K, N, group_size, _stream(c.device)),
          "q4_quantize_groupwise")
    return packed, scales


def q4_dequantize_groupwise(packed, scales, group_size: int, ctx=None):
    c = _ctx_for(packed, ctx)
    K, N = packed.shape[0] * 2, packed.shape[1]
    dst = torch.empty((K, N), dtype=torch.float32, device=packed.device)
    check(c.lib.lhb_q4_dequantize_groupwise(c.handle, _t(packed, torch.uint8, "packed"),
                                            _t(scales, torch.float32, "scales"), dst.data_ptr(), K,
                                            N, group_size, _stream(c.device)),
          "q4_dequantize_groupwise")
    return dst


# ---------------------------------------------------------------------------
# GEMMs  (src/kernels/gemm_quant.hpp:42-57)
# ---------------------------------------------------------------------------

def _out(C_, M, N, like, beta):
    if C_ is None:
        if beta != 0.0:
            raise ValueError("beta != 0 needs C")
        return torch.empty((M, N), dtype=torch.float32, device=like.device)
    if tuple(C_.shape) != (M, N):
        raise ValueError(f"C has shape {tuple(C_.shape)}, expected {(M, N)}")
    return C_


def gemm_w8a8(A_q, B_q, A_scales, B_scales, C=None, alpha: float = 1.0, beta: float = 0.0, ctx=None):
    """C = beta*C + alpha * A_scales[m] * B_scales[n] * (A_q @ B_q), int32 accumulate."""
    c = _ctx_for(A_q, ctx)
    M, K = A_q.shape
    K2, N = B_q.shape
    if K2 != K:
        raise ValueError("inner dimensions differ")
    out = _out(C, M, N, A_q, beta)
    check(c.lib.lhb_gemm_w8a8(c.handle, _t(A_q, torch.int8, "A_q"), _t(B_q, torch.int8, "B_q"),
                              _t(A_scales, torch.float32, "A_scales"),
                              _t(B_scales, torch.float32, "B_scales"),
                              _t(out, torch.float32, "C"), M, N, K, alpha, beta, _stream(c.device)),
          "gemm_w8a8")
    return out


def gemm_w4a16_groupwise(A, B_packed, B_scales, group_size: int, C=None, alpha: float = 1.0,
                         beta: float = 0.0, ctx=None):
    """C = beta*C + alpha * A @ dequant(B_packed, B_scales); fp32 A [M, K], packed [K/2, N]."""
    c = _ctx_for(A, ctx)
    M, K = A.shape
    N = B_packed.shape[1]
    if B_packed.shape[0] * 2 != K:
        raise ValueError("packed rows must be K/2")
    out = _out(C, M, N, A, beta)
    check(c.lib.lhb_gemm_w4a16_groupwise(c.handle, _t(A, torch.float32, "A"),
                                         _t(B_packed, torch.uint8, "B_packed"),
                                         _t(B_scales, torch.float32, "B_scales"),
                                         _t(out, torch.float32, "C"), M, N, K, group_size, alpha,
                                         beta, _stream(c.device)), "gemm_w4a16_groupwise")
    return out


def gemm_w8a16_perchannel(A, B_q, B_scales, C=None, alpha: float = 1.0, beta: float = 0.0, ctx=None):
    """Weight-only int8: C = beta*C + alpha * A @ (B_q * B_scales[n])."""
    c = _ctx_for(A, ctx)
    M, K = A.shape
    N = B_q.shape[1]
    if B_q.shape[0] != K:
        raise ValueError("inner dimensions differ")
    out = _out(C, M, N, A, beta)
    check(c.lib.lhb_gemm_w8a16_perchannel(c.handle, _t(A, torch.float32, "A"),
                                          _t(B_q, torch.int8, "B_q"),
                                          _t(B_scales, torch.float32, "B_scales"),
                                          _t(out, torch.float32, "C"), M, N, K, alpha, beta,
                                          _stream(c.device)), "gemm_w8a16_perchannel")
    return out


# ---------------------------------------------------------------------------
# paged KV cache  (src/kernels/kvcache.hpp, kvcache_quant.hpp)
# ---------------------------------------------------------------------------

def paged_kv_append_q8(k_pool, v_pool, k_scales, v_scales, k_new, v_new, block_table,
                       L: PagedLayout, past_len: int, seq_new: int, ctx=None):
    c = _ctx_for(k_pool, ctx)
    check(c.lib.lhb_paged_kv_append_q8(
        c.handle, _t(k_pool, torch.int8, "k_pool"), _t(v_pool, torch.int8, "v_pool"),
        _t(k_scales, torch.float32, "k_scales"), _t(v_scales, torch.float32, "v_scales"),
        _t(k_new, torch.float32, "k_new"), _t(v_new, torch.float32, "v_new"),
        _t(block_table, torch.int32, "block_table"), C.byref(L), past_len, seq_new,
        _stream(c.device)), "paged_kv_append_q8")


def paged_kv_append_q8_batched(k_pool, v_pool, k_scales, v_scales, k_new, v_new, block_tables,
                               past_lens, L: PagedLayout, seq_new: int = 1, ctx=None):
    c = _ctx_for(k_pool, ctx)
    n_req, max_blocks = block_tables.shape
    check(c.lib.lhb_paged_kv_append_q8_batched(
        c.handle, _t(k_pool, torch.int8, "k_pool"), _t(v_pool, torch.int8, "v_pool"),
        _t(k_scales, torch.float32, "k_scales"), _t(v_scales, torch.float32, "v_scales"),
        _t(k_new, torch.float32, "k_new"), _t(v_new, torch.float32, "v_new"),
        _t(block_tables, torch.int32, "block_tables"), max_blocks,
        _t(past_lens, torch.int32, "past_lens"), n_req, C.byref(L), seq_new, _stream(c.device)),
        "paged_kv_append_q8_batched")


def paged_kv_append(k_pool, v_pool, k_new, v_new, block_table, L: PagedLayout, past_len: int,
                    seq_new: int, ctx=None):
    """fp32 pools (src/kernels/kvcache.hpp:50-55)."""
    c = _ctx_for(k_pool, ctx)
    check(c.lib.lhb_paged_kv_append_f32(
        c.handle, _t(k_pool, torch.float32, "k_pool"), _t(v_pool, torch.float32, "v_pool"),
        _t(k_new, torch.float32, "k_new"), _t(v_new, torch.float32, "v_new"),
        _t(block_table, torch.int32, "block_table"), C.byref(L), past_len, seq_new,
        _stream(c.device)), "paged_kv_append")


# ---------------------------------------------------------------------------
# paged attention  (src/kernels/kvcache_quant.hpp:51-57, paged_attention.hpp:42-63)
# ---------------------------------------------------------------------------

def paged_attention_q8(Q, K_pool, V_pool, K_scales, V_scales, block_table, seq_len: int,
                       cfg: PagedAttnCfg, L: PagedLayout, O=None, ctx=None):
    """Single request: Q/O [n_q_heads, seq_q, head_dim]."""
    c = _ctx_for(Q, ctx)
    O = torch.empty_like(Q) if O is None else O
    check(c.lib.lhb_paged_attention_q8(
        c.handle, _t(Q, torch.float32, "Q"), _t(K_pool, torch.int8, "K_pool"),
        _t(V_pool, torch.int8, "V_pool"), _t(K_scales, torch.float32, "K_scales"),
        _t(V_scales, torch.float32, "V_scales"), _t(block_table, torch.int32, "block_table"),
        seq_len, _t(O, torch.float32, "O"), C.byref(cfg), C.byref(L), _stream(c.device)),
        "paged_attention_q8")
    return O


def paged_attention_q8_batched(Q, K_pool, V_pool, K_scales, V_scales, block_tables, seq_lens,
                               cfg: PagedAttnCfg, L: PagedLayout, O=None, ctx=None):
    """Q/O [n_requests, n_q_heads, seq_q, head_dim]; tables [n_requests, max_blocks] int32."""
    c = _ctx_for(Q, ctx)
    O = torch.empty_like(Q) if O is None else O
    n_req, max_blocks = block_tables.shape
    check(c.lib.lhb_paged_attention_q8_batched(
        c.handle, _t(Q, torch.float32, "Q"), _t(K_pool, torch.int8, "K_pool"),
        _t(V_pool, torch.int8, "V_pool"), _t(K_scales, torch.float32, "K_scales"),
        _t(V_scales, torch.float32, "V_scales"), _t(block_tables, torch.int32, "block_tables"),
        max_blocks, _t(seq_lens, torch.int32, "seq_lens"), n_req, _t(O, torch.float32, "O"),
        C.byref(cfg), C.byref(L), _stream(c.device)), "paged_attention_q8_batched")
    return O


def paged_attention_batched_f32(Q, K_pool, V_pool, block_tables, seq_lens, cfg: PagedAttnCfg,
                                L: PagedLayout, O=None, ctx=None):
    """fp32 pools, lh::paged_attention_batched (src/kernels/paged_attention.hpp:50-63)."""
    c = _ctx_for(Q, ctx)
    O = torch.empty_like(Q) if O is None else O
    n_req, max_blocks = block_tables.shape
    check(c.lib.lhb_paged_attention_f32_batched(
        c.handle, _t(Q, torch.float32, "Q"), _t(K_pool, torch.float32, "K_pool"),
        _t(V_pool, torch.float32, "V_pool"), _t(block_tables, torch.int32, "block_tables"),
        max_blocks, _t(seq_lens, torch.int32, "seq_lens"), n_req, _t(O, torch.float32, "O"),
        C.byref(cfg), C.byref(L), _stream(c.device)), "paged_attention_batched_f32")
    return O


def paged_attention_q8_batched_noalloc(Q, K_pool, V_pool, K_scales, V_scales, block_tables, seq_lens,
                                       cfg: PagedAttnCfg, L: PagedLayout, O):
    """Batched int8 decode attention through the entry point that allocates no
    device memory and takes no context (its scratch is a fixed array inside the
    library).  For hosts that must not allocate: every buffer, the output
    included, is supplied by the caller.  Limits and the sharing rule are stated
    with the declaration in include/lhb200.h."""
    lib = _cabi.load()
    n_req, max_blocks = block_tables.shape
    dev = Q.device.index
    check(lib.lhb_paged_attention_q8_batched_noalloc(
        _t(Q, torch.float32, "Q"), _t(K_pool, torch.int8, "K_pool"), _t(V_pool, torch.int8, "V_pool"),
        _t(K_scales, torch.float32, "K_scales"), _t(V_scales, torch.float32, "V_scales"),
        _t(block_tables, torch.int32, "block_tables"), max_blocks, _t(seq_lens, torch.int32, "seq_lens"),
        n_req, _t(O, torch.float32, "O"), C.byref(cfg), C.byref(L), _stream(dev)),
        "paged_attention_q8_batched_noalloc")
    return O


# ---- decode-step glue -----------------------------------------------------------

def rmsnorm(x, gamma, eps: float = 1e-5, out=None, ctx=None):
    """lh::rmsnorm (src/kernels/normalization.hpp:21): fp32 [rows, dim] -> [rows, dim]."""
    c = _ctx_for(x, ctx)
    rows, dim = x.shape
    y = torch.empty_like(x) if out is None else out
    check(c.lib.lhb_rmsnorm(c.handle, _t(x, torch.float32, "x"), _t(gamma, torch.float32, "gamma"),
                            _t(y, torch.float32, "out"), rows, dim, C.c_float(eps), _stream(c.device)),
          "rmsnorm")
    return y


def rope(x, theta_base: float = 10000.0, freq_scale: float = 1.0, interleaved: bool = True,
         pos_offset: int = 0, ctx=None):
    """lh::rope (src/kernels/rope.hpp:19-21), in place on fp32 [seq, n_heads, head_dim]."""
    c = _ctx_for(x, ctx)
    seq, n_heads, head_dim = x.shape
    check(c.lib.lhb_rope(c.handle, _t(x, torch.float32, "x"), seq, n_heads, head_dim,
                         C.c_float(theta_base), C.c_float(freq_scale), int(bool(interleaved)),
                         int(pos_offset), _stream(c.device)), "rope")
    return x


def rope_decode_batched(x, positions, theta_base: float = 10000.0, freq_scale: float = 1.0,
                        interleaved: bool = True, ctx=None):
    """One token per request: fp32 [n_req, n_heads, head_dim] rotated in place at positions[r]."""
    c = _ctx_for(x, ctx)
    n_req, n_heads, head_dim = x.shape
    check(c.lib.lhb_rope_decode_batched(c.handle, _t(x, torch.float32, "x"),
                                        _t(positions, torch.int32, "positions"), n_req, n_heads,
                                        head_dim, C.c_float(theta_base), C.c_float(freq_scale),
                                        int(bool(interleaved)), _stream(c.device)), "rope_decode_batched")
    return x


def gemm_w4a16_norm(x, gamma, eps: float, B_packed, B_scales, group_size: int, C=None, alpha: float = 1.0,
                    beta: float = 0.0, scratch=None, ctx=None):
    """C = beta*C + alpha * rmsnorm(x, gamma, eps) @ dequant(B): one fused call where the library serves
    the shape, else lhb_rmsnorm into `scratch` ([M, K], allocated if None) and the plain GEMM."""
    c = _ctx_for(x, ctx)
    M, K_ = x.shape
    N = B_packed.shape[1]
    out = _out(C, M, N, x, beta)
    rc = c.lib.lhb_gemm_w4a16_groupwise_prologue(
        c.handle, _t(x, torch.float32, "x"), 1, _t(gamma, torch.float32, "gamma"), float(eps),
        _t(B_packed, torch.uint8, "B_packed"), _t(B_scales, torch.float32, "B_scales"), _t(out, torch.float32, "C"),
        M, N, K_, group_size, alpha, beta, _stream(c.device))
    if rc == _cabi.ERR_UNSUPPORTED:
        h = rmsnorm(x, gamma, eps, out=scratch, ctx=ctx)
        return gemm_w4a16_groupwise(h, B_packed, B_scales, group_size, C=out, alpha=alpha, beta=beta, ctx=ctx)
    check(rc, "gemm_w4a16_groupwise_prologue")
    return out


def gemm_w4a16_swiglu(x, B_packed, B_scales, group_size: int, C=None, alpha: float = 1.0, beta: float = 0.0,
                      scratch=None, ctx=None):
    """C = beta*C + alpha * swiglu(x) @ dequant(B) for x = [M, 2K] (gate || value); fused where served."""
    c = _ctx_for(x, ctx)
    M, K2 = x.shape
    K_ = K2 // 2
    N = B_packed.shape[1]
    out = _out(C, M, N, x, beta)
    rc = c.lib.lhb_gemm_w4a16_groupwise_prologue(
        c.handle, _t(x, torch.float32, "x"), 2, None, 0.0, _t(B_packed, torch.uint8, "B_packed"),
        _t(B_scales, torch.float32, "B_scales"), _t(out, torch.float32, "C"), M, N, K_, group_size, alpha, beta,
        _stream(c.device))
    if rc == _cabi.ERR_UNSUPPORTED:
        a = swiglu(x, out=scratch, ctx=ctx)
        return gemm_w4a16_groupwise(a, B_packed, B_scales, group_size, C=out, alpha=alpha, beta=beta, ctx=ctx)
    check(rc, "gemm_w4a16_groupwise_prologue")
    return out


def qkv_rope_append_q8_decode(qkv, q_out, k_pool, v_pool, k_scales, v_scales, block_tables, positions,
                              n_q_heads: int, L: PagedLayout, theta_base: float = 10000.0, freq_scale: float = 1.0,
                              interleaved: bool = True, ctx=None):
    """Split a fused QKV row, rotate q and k at positions[r], write q to `q_out` [n_req, n_q_heads, head_dim] and
    quantise k, v into the paged int8 cache: rope + rope + append in one launch, same bits."""
    c = _ctx_for(qkv, ctx)
    n_req, max_blocks = block_tables.shape
    check(c.lib.lhb_qkv_rope_append_q8_decode(
        c.handle, _t(qkv, torch.float32, "qkv"), qkv.stride(0), _t(q_out, torch.float32, "q_out"),
        _t(k_pool, torch.int8, "k_pool"), _t(v_pool, torch.int8, "v_pool"), _t(k_scales, torch.float32, "k_scales"),
        _t(v_scales, torch.float32, "v_scales"), _t(block_tables, torch.int32, "block_tables"), max_blocks,
        _t(positions, torch.int32, "positions"), n_req, n_q_heads, C.byref(L), C.c_float(theta_base),
        C.c_float(freq_scale), int(bool(interleaved)), _stream(c.device)), "qkv_rope_append_q8_decode")
    return q_out


def swiglu(x, out=None, ctx=None):
    """lh::swiglu (src/kernels/activation.hpp:34): fp32 [rows, 2*dim] (gate || value) -> [rows, dim]."""
    c = _ctx_for(x, ctx)
    rows, dim2 = x.shape
    y = torch.empty((rows, dim2 // 2), dtype=torch.float32, device=x.device) if out is None else out
    check(c.lib.lhb_swiglu(c.handle, _t(x, torch.float32, "x"), _t(y, torch.float32, "out"), rows,
                           dim2 // 2, _stream(c.device)), "swiglu")
    return y


# ---- asymmetric int4 (fp16 scale and zero-point per group) ------------------------------

def q4a_quantize_groupwise(src, group_size: int, ctx=None):
    """fp32 [K, N] -> (uint8 packed [K/2, N], fp16 scales [K/G, N], fp16 zero-points [K/G, N])."""
    c = _ctx_for(src, ctx)
    K_, N = src.shape
    packed = torch.empty((K_ // 2, N), dtype=torch.uint8, device=src.device)
    scales = torch.empty((K_ // group_size, N), dtype=torch.float16, device=src.device)
    zeros = torch.empty((K_ // group_size, N), dtype=torch.float16, device=src.device)
    check(c.lib.lhb_q4a_quantize_groupwise(c.handle, _t(src, torch.float32, "src"), packed.data_ptr(),
                                           scales.data_ptr(), zeros.data_ptr(), K_, N, group_size,
                                           _stream(c.device)), "q4a_quantize_groupwise")
    return packed, scales, zeros


def q4a_dequantize_groupwise(packed, scales, zeros, group_size: int, ctx=None):
    c = _ctx_for(packed, ctx)
    K_, N = packed.shape[0] * 2, packed.shape[1]
    dst = torch.empty((K_, N), dtype=torch.float32, device=packed.device)
    check(c.lib.lhb_q4a_dequantize_groupwise(c.handle, _t(packed, torch.uint8, "packed"),
                                             _t(scales, torch.float16, "scales"), _t(zeros, torch.float16, "zeros"),
                                             dst.data_ptr(), K_, N, group_size, _stream(c.device)),
          "q4a_dequantize_groupwise")
    return dst


def gemm_w4a16_asym(A, B_packed, B_scales, B_zeros, group_size: int, C=None, alpha: float = 1.0,
                    beta: float = 0.0, ctx=None):
    """C = beta*C + alpha * A @ ((u - zero) * scale); fp32 A [M, K], packed [K/2, N], fp16 parameters."""
    c = _ctx_for(A, ctx)
    M, K_ = A.shape
    N = B_packed.shape[1]
    if B_packed.shape[0] * 2 != K_:
        raise ValueError("packed rows must be K/2")
    out = _out(C, M, N, A, beta)
    check(c.lib.lhb_gemm_w4a16_asym(c.handle, _t(A, torch.float32, "A"), _t(B_packed, torch.uint8, "B_packed"),
                                    _t(B_scales, torch.float16, "B_scales"), _t(B_zeros, torch.float16, "B_zeros"),
                                    _t(out, torch.float32, "C"), M, N, K_, group_size, alpha, beta,
                                    _stream(c.device)), "gemm_w4a16_asym")
    return out


# ---- FP8 E4M3 ----------------------------------------------------------------------------

def fp8_quantize_per_tensor(src, ctx=None):
    """fp32 tensor -> (uint8 E4M3 bytes of the same shape, fp32 scale as a 1-element CUDA tensor)."""
    c = _ctx_for(src, ctx)
    dst = torch.empty(src.shape, dtype=torch.uint8, device=src.device)
    scale = torch.empty(1, dtype=torch.float32, device=src.device)
    check(c.lib.lhb_fp8_quantize_per_tensor(c.handle, _t(src, torch.float32, "src"), dst.data_ptr(),
                                            scale.data_ptr(), src.numel(), _stream(c.device)),
          "fp8_quantize_per_tensor")
    return dst, scale


def fp8_quantize_per_row(src, ctx=None):
    c = _ctx_for(src, ctx)
    rows, dim = src.shape
    dst = torch.empty((rows, dim), dtype=torch.uint8, device=src.device)
    scales = torch.empty(rows, dtype=torch.float32, device=src.device)
    check(c.lib.lhb_fp8_quantize_per_row(c.handle, _t(src, torch.float32, "src"), dst.data_ptr(),
                                         scales.data_ptr(), rows, dim, _stream(c.device)), "fp8_quantize_per_row")
    return dst, scales


def fp8_quantize_per_col(src, ctx=None):
    c = _ctx_for(src, ctx)
    rows, cols = src.shape
    dst = torch.empty((rows, cols), dtype=torch.uint8, device=src.device)
    scales = torch.empty(cols, dtype=torch.float32, device=src.device)
    check(c.lib.lhb_fp8_quantize_per_col(c.handle, _t(src, torch.float32, "src"), dst.data_ptr(),
                                         scales.data_ptr(), rows, cols, _stream(c.device)), "fp8_quantize_per_col")
    return dst, scales


def fp8_dequantize(src, scales, mode: int, ctx=None):
    """mode 0: one scale (1-element tensor), 1: per row, 2: per column."""
    c = _ctx_for(src, ctx)
    rows, cols = src.shape
    dst = torch.empty((rows, cols), dtype=torch.float32, device=src.device)
    check(c.lib.lhb_fp8_dequantize(c.handle, _t(src, torch.uint8, "src"), _t(scales, torch.float32, "scales"),
                                   dst.data_ptr(), rows, cols, int(mode), _stream(c.device)), "fp8_dequantize")
    return dst


def gemm_fp8_e4m3(A, B, A_scale: float, B_scale: float, C=None, alpha: float = 1.0, beta: float = 0.0, ctx=None):
    """lh::gemm_fp8_e4m3: A [M, K], B [K, N] uint8 E4M3 bytes, per-tensor scales as Python floats."""
    c = _ctx_for(A, ctx)
    M, K_ = A.shape
    N = B.shape[1]
    out = _out(C, M, N, A, beta)
    check(c.lib.lhb_gemm_fp8_e4m3(c.handle, _t(A, torch.uint8, "A"), _t(B, torch.uint8, "B"), float(A_scale),
                                  float(B_scale), _t(out, torch.float32, "C"), M, N, K_, alpha, beta,
                                  _stream(c.device)), "gemm_fp8_e4m3")
    return out

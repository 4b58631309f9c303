"""ctypes front end to the two CPU checkers under ``oracle/``.

``Checker("lho")`` drives the C restatement (``oracle/_build/liblh_oracle.so``,
compiled on demand with gcc); ``Checker("lhr")`` drives the reference's own
compiled sources (``oracle/_ref/liblh_ref.so``), which exists only where it was
built from a reference checkout.  Both export the same functions under the two
prefixes, so every method below works on either.

Test infrastructure only: the product package never imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
PORT_SO = os.path.join(ORACLE_DIR, "_build", "liblh_oracle.so")
REF_SO = os.path.join(ORACLE_DIR, "_ref", "liblh_ref.so")


class Layout(C.Structure):
    """Mirror of the paged-cache layout struct (num_blocks, block_size, n_kv_heads, head_dim)."""
    _fields_ = [("num_blocks", C.c_int), ("block_size", C.c_int),
                ("n_kv_heads", C.c_int), ("head_dim", C.c_int)]


class AttnCfg(C.Structure):
    """Mirror of the paged-attention config struct; ``causal`` is an int (0/1)."""
    _fields_ = [("n_q_heads", C.c_int), ("n_kv_heads", C.c_int), ("seq_q", C.c_int),
                ("head_dim", C.c_int), ("causal", C.c_int), ("scale", C.c_float),
                ("window", C.c_int), ("chunk", C.c_int)]


def build_port(force: bool = False) -> str:
    """Compile the C restatement if the shared object is missing or stale."""
    src = os.path.join(ORACLE_DIR, "lh_oracle.c")
    if force or not os.path.exists(PORT_SO) or os.path.getmtime(PORT_SO) < os.path.getmtime(src):
        os.makedirs(os.path.dirname(PORT_SO), exist_ok=True)
        subprocess.check_call(["gcc", "-std=c11", "-O3", "-fPIC", "-fopenmp", "-fvisibility=hidden",
                               "-shared", "-o", PORT_SO, src, "-lm"])
    return PORT_SO


def ref_available() -> bool:
    return os.path.exists(REF_SO)


def _p(a, dtype=None):
    if a is None:
        return None
    if dtype is not None:
        assert a.dtype == dtype, (a.dtype, dtype)
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.c_void_p)


@dataclass
class PagedPools:
    k: np.ndarray
    v: np.ndarray
    ks: np.ndarray
    vs: np.ndarray


class Checker:
    def __init__(self, prefix: str = "lho"):
        assert prefix in ("lho", "lhr")
        self.prefix = prefix
        path = build_port() if prefix == "lho" else REF_SO
        self.lib = C.CDLL(path)
        self.kind = "port" if prefix == "lho" else "reference"

    def fn(self, name, restype=None):
        f = getattr(self.lib, f"{self.prefix}_{name}")
        f.restype = restype
        return f

    # -- scalar helpers -------------------------------------------------
    def round_to_bf16(self, x: np.ndarray) -> np.ndarray:
        y = np.ascontiguousarray(x, dtype=np.float32).copy()
        self.fn("round_to_bf16")(_p(y), C.c_int64(y.size))
        return y

    def max_threads(self) -> int:
        return int(self.fn("max_threads", C.c_int)())

    def set_threads(self, n: int) -> None:
        """Thread count of the `par_*` harness loops (overrides OMP_NUM_THREADS)."""
        self.fn("set_threads")(int(n))

    # -- quantisers -----------------------------------------------------
    def q8_quantize_per_tensor(self, x):
        q = np.empty(x.shape, np.int8)
        s = np.empty(1, np.float32)
        self.fn("q8_quantize_per_tensor")(_p(x, np.float32), _p(q), _p(s), C.c_int64(x.size))
        return q, s

    def q8_dequantize_per_tensor(self, q, scale):
        d = np.empty(q.shape, np.float32)
        self.fn("q8_dequantize_per_tensor")(_p(q, np.int8), C.c_float(float(scale)), _p(d), C.c_int64(q.size))
        return d

    def q8_quantize_per_row(self, x):
        rows, dim = x.shape
        q = np.empty((rows, dim), np.int8)
        s = np.empty(rows, np.float32)
        self.fn("q8_quantize_per_row")(_p(x, np.float32), _p(q), _p(s), rows, dim)
        return q, s

    def q8_dequantize_per_row(self, q, s):
        rows, dim = q.shape
        d = np.empty((rows, dim), np.float32)
        self.fn("q8_dequantize_per_row")(_p(q, np.int8), _p(s, np.float32), _p(d), rows, dim)
        return d

    def q8_quantize_per_col(self, x):
        rows, cols = x.shape
        q = np.empty((rows, cols), np.int8)
        s = np.empty(cols, np.float32)
        self.fn("q8_quantize_per_col")(_p(x, np.float32), _p(q), _p(s), rows, cols)
        return q, s

    def q8_dequantize_per_col(self, q, s):
        rows, cols = q.shape
        d = np.empty((rows, cols), np.float32)
        self.fn("q8_dequantize_per_col")(_p(q, np.int8), _p(s, np.float32), _p(d), rows, cols)
        return d

    def q4_quantize_groupwise(self, w, G):
        K, N = w.shape
        p = np.empty((K // 2, N), np.uint8)
        s = np.empty((K // G, N), np.float32)
        self.fn("q4_quantize_groupwise")(_p(w, np.float32), _p(p), _p(s), K, N, G)
        return p, s

    def q4_dequantize_groupwise(self, p, s, G):
        K, N = p.shape[0] * 2, p.shape[1]
        d = np.empty((K, N), np.float32)
        self.fn("q4_dequantize_groupwise")(_p(p, np.uint8), _p(s, np.float32), _p(d), K, N, G)
        return d

    def q4_get(self, p, k, n):
        return int(self.fn("q4_get", C.c_int)(_p(p, np.uint8), k, n, p.shape[1]))

    # -- GEMMs ------------------------------------------------------------
    def gemm_f32(self, A, B, C0=None, alpha=1.0, beta=0.0):
        M, K = A.shape
        N = B.shape[1]
        out = np.zeros((M, N), np.float32) if C0 is None else C0.copy()
        self.fn("gemm_f32")(_p(A, np.float32), _p(B, np.float32), _p(out), M, N, K,
                            C.c_float(alpha), C.c_float(beta))
        return out

    def gemm_w8a8(self, Aq, Bq, a_s, b_s, C0=None, alpha=1.0, beta=0.0):
        M, K = Aq.shape
        N = Bq.shape[1]
        out = np.zeros((M, N), np.float32) if C0 is None else C0.copy()
        self.fn("gemm_w8a8")(_p(Aq, np.int8), _p(Bq, np.int8), _p(a_s, np.float32),
                             _p(b_s, np.float32), _p(out), M, N, K, C.c_float(alpha), C.c_float(beta))
        return out

    def gemm_w4a16_groupwise(self, A, Bp, Bs, G, C0=None, alpha=1.0, beta=0.0):
        M, K = A.shape
        N = Bp.shape[1]
        out = np.zeros((M, N), np.float32) if C0 is None else C0.copy()
        self.fn("gemm_w4a16_groupwise")(_p(A, np.float32), _p(Bp, np.uint8), _p(Bs, np.float32),
                                        _p(out), M, N, K, G, C.c_float(alpha), C.c_float(beta))
        return out

    def gemm_w8a16_perchannel(self, A, Bq, Bs, C0=None, alpha=1.0, beta=0.0):
        M, K = A.shape
        N = Bq.shape[1]
        out = np.zeros((M, N), np.float32) if C0 is None else C0.copy()
        self.fn("gemm_w8a16_perchannel")(_p(A, np.float32), _p(Bq, np.int8), _p(Bs, np.float32),
                                         _p(out), M, N, K, C.c_float(alpha), C.c_float(beta))
        return out

    # -- FP8 E4M3 -----------------------------------------------------------
    def f32_to_e4m3_bits(self, x):
        f = self.fn("f32_to_e4m3_bits", C.c_uint8)
        return np.array([f(C.c_float(float(v))) for v in np.asarray(x, np.float32).ravel()], np.uint8)

    def e4m3_bits_to_f32(self, b):
        f = self.fn("e4m3_bits_to_f32", C.c_float)
        return np.array([f(C.c_uint8(int(v))) for v in np.asarray(b, np.uint8).ravel()], np.float32)

    def fp8_quantize_per_tensor(self, x):
        x = np.ascontiguousarray(x, np.float32)
        q = np.zeros(x.shape, np.uint8)
        s = np.zeros(1, np.float32)
        self.fn("fp8_quantize_per_tensor")(_p(x), _p(q), _p(s), C.c_int64(x.size))
        return q, float(s[0])

    def fp8_quantize_per_row(self, x):
        x = np.ascontiguousarray(x, np.float32)
        q = np.zeros(x.shape, np.uint8)
        s = np.zeros(x.shape[0], np.float32)
        self.fn("fp8_quantize_per_row")(_p(x), _p(q), _p(s), x.shape[0], x.shape[1])
        return q, s

    def fp8_quantize_per_col(self, x):
        x = np.ascontiguousarray(x, np.float32)
        q = np.zeros(x.shape, np.uint8)
        s = np.zeros(x.shape[1], np.float32)
        self.fn("fp8_quantize_per_col")(_p(x), _p(q), _p(s), x.shape[0], x.shape[1])
        return q, s

    def fp8_dequantize(self, q, scales, mode):
        """mode 0: one scale, 1: per row, 2: per column."""
        q = np.ascontiguousarray(q, np.uint8)
        d = np.zeros(q.shape, np.float32)
        sc = np.ascontiguousarray(np.atleast_1d(np.asarray(scales, np.float32)))
        self.fn("fp8_dequantize")(_p(q), _p(sc), _p(d), q.shape[0], q.shape[1], int(mode))
        return d

    def gemm_fp8_e4m3(self, A, B, a_scale, b_scale, C0=None, alpha=1.0, beta=0.0):
        M, K = A.shape
        N = B.shape[1]
        out = np.zeros((M, N), np.float32) if C0 is None else C0.copy()
        self.fn("gemm_fp8_e4m3")(_p(A, np.uint8), _p(B, np.uint8), C.c_float(a_scale), C.c_float(b_scale), _p(out),
                                 M, N, K, C.c_float(alpha), C.c_float(beta))
        return out

    # -- asymmetric int4 (extension; the compiled reference has no such scheme) ----------
    def f32_to_f16_bits(self, x):
        f = self.fn("f32_to_f16_bits", C.c_uint16)
        return np.array([f(C.c_float(float(v))) for v in np.asarray(x, np.float32).ravel()], np.uint16)

    def q4a_quantize_groupwise(self, w, G):
        w = np.ascontiguousarray(w, np.float32)
        K, N = w.shape
        p = np.zeros((K // 2, N), np.uint8)
        s = np.zeros((K // G, N), np.uint16)
        z = np.zeros((K // G, N), np.uint16)
        self.fn("q4a_quantize_groupwise")(_p(w), _p(p), _p(s), _p(z), K, N, G)
        return p, s.view(np.float16), z.view(np.float16)

    def q4a_dequantize_groupwise(self, p, s, z, G):
        K, N = p.shape[0] * 2, p.shape[1]
        d = np.zeros((K, N), np.float32)
        self.fn("q4a_dequantize_groupwise")(_p(p, np.uint8), _p(s.view(np.uint16)), _p(z.view(np.uint16)), _p(d), K, N, G)
        return d

    def gemm_w4a16_asym(self, A, Bp, Bs, Bz, G, C0=None, alpha=1.0, beta=0.0):
        M, K = A.shape
        N = Bp.shape[1]
        out = np.zeros((M, N), np.float32) if C0 is None else C0.copy()
        self.fn("gemm_w4a16_asym")(_p(A, np.float32), _p(Bp, np.uint8), _p(Bs.view(np.uint16)),
                                   _p(Bz.view(np.uint16)), _p(out), M, N, K, G, C.c_float(alpha), C.c_float(beta))
        return out

    # -- decode-step glue ---------------------------------------------------
    def rmsnorm(self, x, gamma, eps=1e-5):
        x = np.ascontiguousarray(x, np.float32)
        rows, dim = x.shape
        y = np.empty_like(x)
        self.fn("rmsnorm")(_p(x), _p(gamma, np.float32), _p(y), rows, dim, C.c_float(eps))
        return y

    def rope(self, x, theta_base=10000.0, freq_scale=1.0, interleaved=True, pos_offset=0):
        """x: [seq, n_heads, head_dim]; returns the rotated copy."""
        y = np.ascontiguousarray(x, np.float32).copy()
        seq, n_heads, head_dim = y.shape
        self.fn("rope")(_p(y), seq, n_heads, head_dim, C.c_float(theta_base), C.c_float(freq_scale),
                        int(bool(interleaved)), int(pos_offset))
        return y

    def swiglu(self, x):
        x = np.ascontiguousarray(x, np.float32)
        rows, dim2 = x.shape
        y = np.empty((rows, dim2 // 2), np.float32)
        self.fn("swiglu")(_p(x), _p(y), rows, dim2 // 2)
        return y

    # -- paged KV -----------------------------------------------------------
    @staticmethod
    def empty_pools_q8(L: Layout) -> PagedPools:
        shp = (L.num_blocks, L.n_kv_heads, L.block_size, L.head_dim)
        return PagedPools(np.zeros(shp, np.int8), np.zeros(shp, np.int8),
                          np.zeros(shp[:3], np.float32), np.zeros(shp[:3], np.float32))

    def paged_kv_append_q8(self, pools: PagedPools, k_new, v_new, table, L, past_len, seq_new):
        self.fn("paged_kv_append_q8")(_p(pools.k, np.int8), _p(pools.v, np.int8),
                                      _p(pools.ks, np.float32), _p(pools.vs, np.float32),
                                      _p(k_new, np.float32), _p(v_new, np.float32),
                                      _p(table, np.int32), C.byref(L), past_len, seq_new)

    def paged_kv_append_f32(self, k_pool, v_pool, k_new, v_new, table, L, past_len, seq_new):
        self.fn("paged_kv_append_f32")(_p(k_pool, np.float32), _p(v_pool, np.float32),
                                       _p(k_new, np.float32), _p(v_new, np.float32),
                                       _p(table, np.int32), C.byref(L), past_len, seq_new)

    def paged_attention_q8(self, Q, pools: PagedPools, table, seq_len, cfg, L):
        O = np.zeros_like(Q)
        self.fn("paged_attention_q8")(_p(Q, np.float32), _p(pools.k), _p(pools.v), _p(pools.ks),
                                      _p(pools.vs), _p(table, np.int32), seq_len, _p(O),
                                      C.byref(cfg), C.byref(L))
        return O

    def paged_attention_f32(self, Q, k_pool, v_pool, table, seq_len, cfg, L):
        O = np.zeros_like(Q)
        self.fn("paged_attention_f32")(_p(Q, np.float32), _p(k_pool, np.float32),
                                       _p(v_pool, np.float32), _p(table, np.int32), seq_len, _p(O),
                                       C.byref(cfg), C.byref(L))
        return O

    def paged_attention_q8_batched(self, Q, pools, tables, seq_lens, cfg, L, parallel=False):
        O = np.zeros_like(Q)
        n_req, max_blocks = tables.shape
        name = "par_paged_attention_q8_batched" if parallel else "paged_attention_q8_batched"
        self.fn(name)(_p(Q, np.float32), _p(pools.k), _p(pools.v), _p(pools.ks), _p(pools.vs),
                      _p(tables, np.int32), max_blocks, _p(seq_lens, np.int32), n_req, _p(O),
                      C.byref(cfg), C.byref(L))
        return O

    def paged_attention_f32_batched(self, Q, k_pool, v_pool, tables, seq_lens, cfg, L):
        O = np.zeros_like(Q)
        n_req, max_blocks = tables.shape
        self.fn("paged_attention_f32_batched")(_p(Q, np.float32), _p(k_pool, np.float32),
                                               _p(v_pool, np.float32), _p(tables, np.int32),
                                               max_blocks, _p(seq_lens, np.int32), n_req, _p(O),
                                               C.byref(cfg), C.byref(L))
        return O

    def paged_kv_append_q8_batched(self, pools, k_new, v_new, new_off, tables, past, seq_new, L):
        n_req, max_blocks = tables.shape
        self.fn("par_paged_kv_append_q8_batched")(
            _p(pools.k), _p(pools.v), _p(pools.ks), _p(pools.vs), _p(k_new, np.float32),
            _p(v_new, np.float32), _p(new_off, np.int64), _p(tables, np.int32), max_blocks,
            _p(past, np.int32), _p(seq_new, np.int32), n_req, C.byref(L))

    # -- bench harness (independent calls over host threads) ----------------
    def par_gemm_w4a16_shards(self, A, Bp_sh, Bs_sh, C_sh, G, alpha=1.0, beta=0.0):
        M, K = A.shape
        n = len(Bp_sh)
        ns = Bp_sh[0].shape[1]
        arr = lambda xs: (C.c_void_p * n)(*[x.ctypes.data for x in xs])
        self.fn("par_gemm_w4a16_shards")(_p(A, np.float32), arr(Bp_sh), arr(Bs_sh), arr(C_sh), M, ns,
                                         K, G, C.c_float(alpha), C.c_float(beta), n)

    def par_gemm_w8a16_shards(self, A, Bq_sh, Bs_sh, C_sh, alpha=1.0, beta=0.0):
        M, K = A.shape
        n = len(Bq_sh)
        ns = Bq_sh[0].shape[1]
        arr = lambda xs: (C.c_void_p * n)(*[x.ctypes.data for x in xs])
        self.fn("par_gemm_w8a16_shards")(_p(A, np.float32), arr(Bq_sh), arr(Bs_sh), arr(C_sh), M, ns,
                                         K, C.c_float(alpha), C.c_float(beta), n)

    def par_gemm_w8a8_mslabs(self, Aq, Bq, a_s, b_s, slab, alpha=1.0, beta=0.0):
        M, K = Aq.shape
        N = Bq.shape[1]
        out = np.zeros((M, N), np.float32)
        self.fn("par_gemm_w8a8_mslabs")(_p(Aq, np.int8), _p(Bq, np.int8), _p(a_s, np.float32),
                                        _p(b_s, np.float32), _p(out), M, N, K, C.c_float(alpha),
                                        C.c_float(beta), slab)
        return out


def best_checker() -> Checker:
    """The reference's compiled code where it exists, else the restatement."""
    return Checker("lhr") if ref_available() else Checker("lho")

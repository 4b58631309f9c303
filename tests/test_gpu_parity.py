"""GPU parity: the CUDA path, called through the C ABI, against
  (1) the committed golden fixtures (outputs of the reference's compiled code),
  (2) the CPU checker on seeded inputs, up to the full benchmark shapes,
  (3) size-independent properties (linearity, shard composition, round trips).
Integer outputs and scales must be bit-identical; fp32 outputs must satisfy
|x - y| <= 1e-4 + 1e-3 |y| (the library tolerance)."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

import golden_io as gio
import longhornai_b200 as lb
from cpu_checker import AttnCfg, Checker, Layout, PagedPools, best_checker
from gpu_util import assert_close, assert_same_bits, dev, host, lb_cfg, lb_layout

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def chk():
    return best_checker()


@pytest.fixture(scope="module")
def lib():
    return lb._cabi.load()


def poll_ok():
    assert lb.default_context().poll() == 0


# --------------------------------------------------------------------------- quantisers

def test_q8_per_row_golden_bits():
    g = gio.load("q8_per_row")
    q, s = lb.q8_quantize_per_row(dev(g["x"]))
    assert_same_bits(host(q), g["q"], "q"); assert_same_bits(host(s), g["s"], "scales")
    assert_same_bits(host(lb.q8_dequantize_per_row(q, s)), g["d"], "dequant")


def test_q8_per_col_golden_bits():
    g = gio.load("q8_per_col")
    q, s = lb.q8_quantize_per_col(dev(g["x"]))
    assert_same_bits(host(q), g["q"], "q"); assert_same_bits(host(s), g["s"], "scales")
    assert_same_bits(host(lb.q8_dequantize_per_col(q, s)), g["d"], "dequant")


@pytest.mark.parametrize("name", gio.names("q4_"))
def test_q4_groupwise_golden_bits(name):
    g = gio.load(name)
    G = int(g["G"])
    p, s = lb.q4_quantize_groupwise(dev(g["w"]), G)
    assert_same_bits(host(p), g["p"], "packed"); assert_same_bits(host(s), g["s"], "scales")
    assert_same_bits(host(lb.q4_dequantize_groupwise(p, s, G)), g["d"], "dequant")


def test_q8_per_tensor_bit_exact(chk):
    """lh::q8_quantize_per_tensor / q8_dequantize_per_tensor (src/kernels/quant.cpp:33-54), incl. the
    all-zero tensor (scale 1) and a size that is no multiple of the block."""
    rng = np.random.default_rng(31)
    for n, mag in ((4000, 3.0), (1, 0.5), (100003, 1e-3), (7, 0.0)):
        x = (rng.uniform(-1, 1, n) * mag).astype(np.float32)
        q, s = lb.q8_quantize_per_tensor(dev(x))
        q0, s0 = chk.q8_quantize_per_tensor(x)
        assert_same_bits(host(q), q0, f"per-tensor q n={n}"); assert_same_bits(host(s), s0, f"per-tensor scale n={n}")
        assert_same_bits(host(lb.q8_dequantize_per_tensor(q, float(s0[0]))), chk.q8_dequantize_per_tensor(q0, s0[0]),
                         f"per-tensor dequant n={n}")
    poll_ok()


def test_quantisers_bit_exact_on_seeded_matrices(chk):
    rng = np.random.default_rng(11)
    x = rng.standard_normal((300, 1000)).astype(np.float32)
    x[17] = 0.0
    x[:, 33] = 0.0
    q, s = lb.q8_quantize_per_row(dev(x)); q0, s0 = chk.q8_quantize_per_row(x)
    assert_same_bits(host(q), q0, "row q"); assert_same_bits(host(s), s0, "row s")
    q, s = lb.q8_quantize_per_col(dev(x)); q0, s0 = chk.q8_quantize_per_col(x)
    assert_same_bits(host(q), q0, "col q"); assert_same_bits(host(s), s0, "col s")
    w = (rng.standard_normal((512, 1000)) * 0.02).astype(np.float32)
    for G in (32, 128):
        p, s = lb.q4_quantize_groupwise(dev(w), G); p0, s0 = chk.q4_quantize_groupwise(w, G)
        assert_same_bits(host(p), p0, f"q4 packed G={G}"); assert_same_bits(host(s), s0, f"q4 scales G={G}")
    poll_ok()


# --------------------------------------------------------------------------- W8A8

def test_w8a8_golden_bits():
    g = gio.load("w8a8_m32n48k64")
    C_ = lb.gemm_w8a8(dev(g["Aq"]), dev(g["Bq"]), dev(g["a_s"]), dev(g["b_s"]))
    assert_same_bits(host(C_), g["C"], "w8a8 beta=0")
    g = gio.load("w8a8_beta")
    C_ = lb.gemm_w8a8(dev(g["Aq"]), dev(g["Bq"]), dev(g["a_s"]), dev(g["b_s"]), C=dev(g["C0"]),
                      alpha=0.5, beta=2.0)
    assert_same_bits(host(C_), g["C"], "w8a8 alpha/beta")


@pytest.mark.parametrize("M,N,K", [(8, 96, 200), (128, 256, 512), (300, 1040, 768), (256, 2048, 1024)])
def test_w8a8_bit_exact_against_checker(chk, lib, M, N, K):
    rng = np.random.default_rng(M + N + K)
    A = rng.standard_normal((M, K)).astype(np.float32)
    W = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    Aq, a_s = chk.q8_quantize_per_row(A)
    Bq, b_s = chk.q8_quantize_per_col(W)
    want = chk.gemm_w8a8(Aq, Bq, a_s, b_s, alpha=1.25)
    got = lb.gemm_w8a8(dev(Aq), dev(Bq), dev(a_s), dev(b_s), alpha=1.25)
    assert_same_bits(host(got), want, f"w8a8 {M}x{N}x{K} fast={lib.lhb_gemm_w8a8_fast_path(M, N, K)}")
    C0 = rng.standard_normal((M, N)).astype(np.float32)
    want = chk.gemm_w8a8(Aq, Bq, a_s, b_s, C0, alpha=0.5, beta=2.0)
    got = lb.gemm_w8a8(dev(Aq), dev(Bq), dev(a_s), dev(b_s), C=dev(C0), alpha=0.5, beta=2.0)
    assert_same_bits(host(got), want, "w8a8 alpha/beta")
    poll_ok()


@pytest.mark.parametrize("M,N,K", [(256, 256, 256), (1024, 2048, 1024), (2048, 4096 + 16, 4096)])
def test_w8a8_cta_pair_path_bit_exact(lib, M, N, K):
    """The CTA-pair kernel (two CTAs share a 256 x 256 tile, used for M >= 256) against the reference
    arithmetic at sizes with many tiles per CTA pair, a ragged last column tile and alpha / beta."""
    port = Checker("lho")
    port.set_threads(len(os.sched_getaffinity(0)))
    rng = np.random.default_rng(7 * M + N + K)
    A = rng.standard_normal((M, K)).astype(np.float32)
    W = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    Aq, a_s = port.q8_quantize_per_row(A)
    Bq, b_s = port.q8_quantize_per_col(W)
    C0 = rng.standard_normal((M, N)).astype(np.float32)
    assert lib.lhb_gemm_w8a8_fast_path(M, N, K) == 1
    got = host(lb.gemm_w8a8(dev(Aq), dev(Bq), dev(a_s), dev(b_s), C=dev(C0), alpha=0.5, beta=2.0))
    poll_ok()
    # the reference's result is C = beta*C0 + (alpha*a_s*b_s)*acc with single roundings: rebuild it from
    # the beta = 0 product of the row-parallel CPU harness
    prod = port.par_gemm_w8a8_mslabs(Aq, Bq, a_s, b_s, 8, alpha=0.5)
    want = (C0 * np.float32(2.0) + prod).astype(np.float32)
    assert_same_bits(got, want, f"pair kernel {M}x{N}x{K}")


def test_w8a8_on_a_limited_number_of_sms_gives_the_same_bits(lib):
    """lhb_ctx_set_sm_limit shrinks the persistent grids (both tcgen05 kernels walk their tiles with a
    stride of the grid size): same result from 148, 37 and 2 SMs; a negative limit is refused."""
    M, N, K = 512, 2048, 1024
    g = torch.Generator(device="cuda").manual_seed(3)
    Aq, a_s = lb.q8_quantize_per_row(torch.randn(M, K, device="cuda", generator=g))
    Bq, b_s = lb.q8_quantize_per_col(torch.randn(K, N, device="cuda", generator=g) * 0.02)
    ctx = lb.default_context()
    full = lb.gemm_w8a8(Aq, Bq, a_s, b_s)
    small = lb.gemm_w8a8(Aq[:100], Bq, a_s[:100], b_s)       # M < 256: the single-CTA kernel
    try:
        for n in (37, 2):
            ctx.set_sm_limit(n)
            assert torch.equal(lb.gemm_w8a8(Aq, Bq, a_s, b_s), full), f"{n} SMs"
            assert torch.equal(lb.gemm_w8a8(Aq[:100], Bq, a_s[:100], b_s), small), f"{n} SMs, single-CTA kernel"
        assert lib.lhb_ctx_set_sm_limit(ctx.handle, -1) != 0
    finally:
        ctx.set_sm_limit(0)
    poll_ok()


@pytest.mark.parametrize("world,M,N_local,K", [(2, 256, 256, 256), (3, 300, 288, 512), (4, 1024, 512, 1024), (8, 640, 160, 384)])
def test_w8a8_sharded_call_fills_every_ranks_matrix(chk, lib, world, M, N_local, K):
    """lhb_gemm_w8a8_sharded, every rank's call issued in turn from one process with all `world`
    full-width matrices in this GPU's memory (the kernel does not know whose memory a destination
    is): afterwards each matrix holds the unsharded product bit for bit, and the guard rows around
    the matrices are untouched (M = 300 and 640 end inside a tile)."""
    rng = np.random.default_rng(world * 1000 + M)
    N = N_local * world
    A = rng.standard_normal((M, K)).astype(np.float32)
    W = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    Aq, a_s = chk.q8_quantize_per_row(A)
    Bq, b_s = chk.q8_quantize_per_col(W)
    want = chk.gemm_w8a8(Aq, Bq, a_s, b_s, alpha=0.75)
    pad = 64                                                  # guard rows before and after every matrix
    mats = [torch.full((M + 2 * pad, N), -7.0, device="cuda") for _ in range(world)]
    full = (C.c_void_p * world)(*[m[pad:].data_ptr() for m in mats])
    dAq, das = dev(Aq), dev(a_s)
    ctx = lb.default_context().handle
    st = torch.cuda.current_stream().cuda_stream
    keep = []
    for rank in range(world):
        Bl = dev(np.ascontiguousarray(Bq[:, rank * N_local:(rank + 1) * N_local]))
        bl = dev(np.ascontiguousarray(b_s[rank * N_local:(rank + 1) * N_local]))
        keep += [Bl, bl]
        rc = lib.lhb_gemm_w8a8_sharded(ctx, dAq.data_ptr(), Bl.data_ptr(), das.data_ptr(), bl.data_ptr(), full, rank,
                                       world, M, N_local, K, 0.75, st)
        assert rc == 0, lib.lhb_status_string(rc)
    poll_ok()
    for r, m in enumerate(mats):
        h = host(m)
        assert_same_bits(h[pad:pad + M], want, f"matrix of rank {r}, world {world}")
        assert (h[:pad] == -7.0).all() and (h[pad + M:] == -7.0).all(), f"rank {r}: rows outside the matrix were written"


def test_w8a8_sharded_call_with_plain_store_push():
    """The same cases with the peer copies written by plain stores instead of bulk stores.  The
    library reads LHB_W8A8_PUSH once per process, so this variant runs in a child process."""
    import subprocess
    import sys
    env = dict(os.environ, LHB_W8A8_PUSH="st")
    r = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-p", "no:cacheprovider", os.path.abspath(__file__), "-k",
                        "test_w8a8_sharded_call_fills_every_ranks_matrix"], env=env, capture_output=True, text=True,
                       timeout=900, cwd=os.path.dirname(os.path.abspath(__file__)))
    assert r.returncode == 0 and "4 passed" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def test_w8a8_sharded_call_rejects_what_it_cannot_push(lib):
    M, K, world = 256, 256, 2
    a = torch.zeros(M, K, dtype=torch.int8, device="cuda")
    s = torch.ones(M, device="cuda")
    ctx = lb.default_context().handle
    for n_local in (144, 48):                                 # fast-path N, but not whole 32-column chunks
        b = torch.zeros(K, n_local, dtype=torch.int8, device="cuda")
        bs = torch.ones(n_local, device="cuda")
        mats = [torch.zeros(M, n_local * world, device="cuda") for _ in range(world)]
        full = (C.c_void_p * world)(*[m.data_ptr() for m in mats])
        rc = lib.lhb_gemm_w8a8_sharded(ctx, a.data_ptr(), b.data_ptr(), s.data_ptr(), bs.data_ptr(), full, 0, world, M,
                                       n_local, K, 1.0, None)
        assert rc != 0 and b"unsupported" in lib.lhb_status_string(rc).lower()
    full = (C.c_void_p * world)(mats[0].data_ptr(), None)
    b = torch.zeros(K, 256, dtype=torch.int8, device="cuda"); bs = torch.ones(256, device="cuda")
    assert lib.lhb_gemm_w8a8_sharded(ctx, a.data_ptr(), b.data_ptr(), s.data_ptr(), bs.data_ptr(), full, 0, world, M, 256, K,
                                     1.0, None) != 0
    assert lib.lhb_gemm_w8a8_sharded(ctx, a.data_ptr(), b.data_ptr(), s.data_ptr(), bs.data_ptr(), full, 2, world, M, 256, K,
                                     1.0, None) != 0
    poll_ok()


# --------------------------------------------------------------------------- W4A16

@pytest.mark.parametrize("name", gio.names("w4a16_"))
def test_w4a16_golden(name):
    g = gio.load(name)
    G = int(g["G"])
    A, p, s = dev(g["A"]), dev(g["p"]), dev(g["s"])
    assert_close(host(lb.gemm_w4a16_groupwise(A, p, s, G)), g["C"], what=name)
    got = lb.gemm_w4a16_groupwise(A, p, s, G, C=dev(g["C0"]), alpha=0.5, beta=2.0)
    assert_close(host(got), g["C_ab"], what=name + " alpha/beta")
    poll_ok()


@pytest.mark.parametrize("M", [1, 2, 3, 5, 8, 13, 16, 17, 32, 40])
@pytest.mark.parametrize("N,K,G", [(1040, 1024, 128), (256, 384, 64), (4096, 2048, 32)])
def test_w4a16_against_checker(chk, lib, M, N, K, G):
    rng = np.random.default_rng(1000 * M + N + K + G)
    A = (rng.standard_normal((M, K)) * rng.choice([1e-3, 1.0, 300.0])).astype(np.float32)
    W = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    p, s = chk.q4_quantize_groupwise(W, G)
    want = chk.gemm_w4a16_groupwise(A, p, s, G)
    got = lb.gemm_w4a16_groupwise(dev(A), dev(p), dev(s), G)
    # tolerance scaled by the magnitude of the activations (the absolute term of
    # the library tolerance is stated for unit-variance activations)
    scale = max(1.0, float(np.abs(A).max()))
    assert_close(host(got) / scale, want / scale,
                 what=f"w4a16 M={M} N={N} K={K} G={G} fast={lib.lhb_gemm_w4a16_fast_path(M, N, K, G)}")
    poll_ok()


def test_w4a16_full_shape_cfg2(chk, lib):
    """Llama-3-8B up-projection shape, M = 1, 8, 32; bf16-stored activations."""
    K, N, G = 4096, 14336, 128
    rng = np.random.default_rng(20242)
    W = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    p, s = lb.q4_quantize_groupwise(dev(W), G)
    p0, s0 = chk.q4_quantize_groupwise(W, G)
    assert_same_bits(host(p), p0, "packed"); assert_same_bits(host(s), s0, "scales")
    for M in (1, 8, 32):
        assert lib.lhb_gemm_w4a16_fast_path(M, N, K, G) == 1
        A = chk.round_to_bf16(rng.standard_normal((M, K)).astype(np.float32))
        got = host(lb.gemm_w4a16_groupwise(dev(A), p, s, G))
        assert_close(got, chk.gemm_w4a16_groupwise(A, p0, s0, G), what=f"cfg2 M={M}")
        # N-shard composition: two compact column shards give the same columns
        h = N // 2
        left = lb.gemm_w4a16_groupwise(dev(A), p[:, :h].contiguous(), s[:, :h].contiguous(), G)
        assert_close(host(left), got[:, :h], rtol=1e-5, atol=1e-6, what="shard composition")
    poll_ok()


@pytest.mark.parametrize("M,N,K,G", [
    (3, 1040, 2048, 128),       # few units: one per CTA, every column tile summed from 16 partials
    (1, 256 * 300, 128, 128),   # K is one unit: every segment is a whole tile, no partials
    (2, 256 * 700, 256, 64),    # ranges of several units: whole tiles in the middle, partial at the ends
    (5, 16 * 37, 4096 + 640, 32),   # ragged N, K not a multiple of the 128-k unit
    (16, 4096, 4096, 256),      # group longer than a unit
    (1, 14336, 4096, 128),      # headline shape: 5 CTAs per column tile
])
def test_w4a16_unit_ranges_and_partial_sums(chk, M, N, K, G):
    """A CTA's contiguous range of work units may cover whole column tiles (written directly)
    and K-slices of tiles (summed through scratch by the last contributor): shapes that hit each
    mix, with alpha/beta, compared with the checker and run twice for determinism."""
    rng = np.random.default_rng(M + N + K)
    A = rng.standard_normal((M, K)).astype(np.float32)
    W = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    p, s = chk.q4_quantize_groupwise(W, G)
    C0 = rng.standard_normal((M, N)).astype(np.float32)
    dA, dp, ds = dev(A), dev(p), dev(s)
    assert lb._cabi.load().lhb_gemm_w4a16_fast_path(M, N, K, G) == 1
    got = lb.gemm_w4a16_groupwise(dA, dp, ds, G, C=dev(C0), alpha=0.5, beta=2.0)
    assert_close(host(got), chk.gemm_w4a16_groupwise(A, p, s, G, C0, alpha=0.5, beta=2.0), what=f"{M}x{N}x{K} G={G}")
    got2 = lb.gemm_w4a16_groupwise(dA, dp, ds, G, C=dev(C0), alpha=0.5, beta=2.0)
    assert torch.equal(got, got2)
    poll_ok()


@pytest.mark.parametrize("M,N,K,G", [(100, 1040, 1024, 128), (300, 512, 2048, 64), (200, 256, 16384, 128)])
def test_w4a16_many_rows_in_slabs(chk, lib, M, N, K, G):
    """More than 64 rows: slabs of 16 rows over one digit pass, or several passes when K is long
    (K = 16384: 80 rows per pass); the last slab is ragged."""
    assert lib.lhb_gemm_w4a16_fast_path(M, N, K, G) == 1
    rng = np.random.default_rng(M + N + K)
    A = rng.standard_normal((M, K)).astype(np.float32)
    W = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    p, s = chk.q4_quantize_groupwise(W, G)
    C0 = rng.standard_normal((M, N)).astype(np.float32)
    got = lb.gemm_w4a16_groupwise(dev(A), dev(p), dev(s), G, C=dev(C0), alpha=0.5, beta=2.0)
    assert_close(host(got), chk.gemm_w4a16_groupwise(A, p, s, G, C0, alpha=0.5, beta=2.0), what=f"{M}x{N}x{K}")
    poll_ok()


@pytest.mark.parametrize("M,N,K,G", [
    (17, 1040, 128, 128),       # one unit per column tile, ragged last tile: every segment whole
    (32, 256, 4096, 128),       # one column tile shared by 32 CTAs: 32 partial slots summed
    (33, 4096, 4096, 256),      # group of two units; second slab holds one row
    (40, 16 * 37, 1024, 128),   # ragged N below three tiles, short second slab
    (64, 6144, 4096, 128),      # two full slabs, whole number of CTAs per tile
    (100, 28672, 512, 128),     # more tiles than three quarters of the SMs: one CTA per tile... or an even deal
    (1024, 512, 256, 128),      # 32 slabs over one digit pass
    (2100, 256, 384, 128),      # three digit passes of up to 1024 rows, short last slab
    (17, 256 * 300, 128, 128),  # more column tiles than CTAs: every CTA walks two whole tiles
    (20, 256 * 200, 384, 128),  # ranges of four or five units over tiles of three: whole and partial segments mixed
])
def test_w4a16_tensor_core_kernel_shapes(chk, M, N, K, G):
    """From 9 rows on gemm_w4a16_groupwise runs on the tensor cores (int8 digits x int8 weights,
    exact int32 sums per group, fp32 fold).  Shapes for each way its work is split, with
    alpha / beta, against the checker, twice for run-to-run determinism."""
    rng = np.random.default_rng(3 * M + N + K + G)
    A = (rng.standard_normal((M, K)) * rng.choice([1e-2, 1.0, 50.0], size=(M, 1))).astype(np.float32)
    W = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    p, s = chk.q4_quantize_groupwise(W, G)
    C0 = rng.standard_normal((M, N)).astype(np.float32)
    dA, dp, ds = dev(A), dev(p), dev(s)
    got = lb.gemm_w4a16_groupwise(dA, dp, ds, G, C=dev(C0), alpha=0.5, beta=2.0)
    want = chk.gemm_w4a16_groupwise(A, p, s, G, C0, alpha=0.5, beta=2.0)
    scale = np.maximum(1.0, np.abs(A).max(axis=1, keepdims=True))     # the absolute term is stated for unit rows
    assert_close(host(got) / scale, want / scale, what=f"tensor-core w4a16 {M}x{N}x{K} G={G}")
    got2 = lb.gemm_w4a16_groupwise(dA, dp, ds, G, C=dev(C0), alpha=0.5, beta=2.0)
    assert torch.equal(got, got2)
    poll_ok()


@pytest.mark.parametrize("knob", ["LHB_W4TC_COOP=0", "LHB_W4TC_SPLIT=1"])
def test_w4a16_tensor_core_kernel_other_hand_offs(knob):
    """The same shapes with the other ways a column tile's partial sums are added up: the last CTA to
    arrive alone (LHB_W4TC_COOP=0) and an even deal of units whatever the tile boundaries
    (LHB_W4TC_SPLIT=1).  The library reads its knobs once per process: child processes."""
    import subprocess
    import sys
    name, value = knob.split("=")
    r = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-p", "no:cacheprovider", os.path.abspath(__file__), "-k",
                        "test_w4a16_tensor_core_kernel_shapes or test_w4a16_with_rmsnorm_and_swiglu_prologue"],
                       env=dict(os.environ, **{name: value}), capture_output=True, text=True, timeout=900,
                       cwd=os.path.dirname(os.path.abspath(__file__)))
    assert r.returncode == 0 and " passed" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def test_w4a16_tensor_core_kernel_is_exact_on_integers():
    """Small integer activations and unit scales: every product and sum is an integer below 2^22 that
    the kernel carries exactly, so the result equals integer arithmetic bit for bit (no tolerance)."""
    M, N, K, G = 32, 512, 512, 128
    rng = np.random.default_rng(77)
    q = rng.integers(-8, 8, size=(K, N)).astype(np.int64)
    a = rng.integers(-1000, 1001, size=(M, K)).astype(np.int64)
    a[:, 0] = 1024                                      # every row's factor is then the same power of two
    packed = ((q[0::2] & 15) | ((q[1::2] & 15) << 4)).astype(np.uint8)
    scales = np.ones((K // G, N), np.float32)
    got = host(lb.gemm_w4a16_groupwise(dev(a.astype(np.float32)), dev(packed), dev(scales), G))
    want = (a @ q).astype(np.float64)
    assert np.abs(want).max() < 2 ** 22
    np.testing.assert_array_equal(got.astype(np.float64), want.astype(np.float32).astype(np.float64))
    poll_ok()


@pytest.mark.parametrize("M", [1, 2, 5, 16, 32])
def test_w4a16_non_finite_activations_are_not_hidden(chk, M):
    """A NaN or an infinity in an activation row makes that row's outputs non-finite, as the
    reference's fp32 accumulation does (src/kernels/gemm_quant.cpp:54-82); the other rows are
    untouched.  (The digit decomposition would otherwise turn NaN into 0 and Inf into a large
    finite number.)"""
    K, N, G = 1024, 1040, 128
    rng = np.random.default_rng(M)
    A = rng.standard_normal((M, K)).astype(np.float32)
    W = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    p, s = chk.q4_quantize_groupwise(W, G)
    clean = chk.gemm_w4a16_groupwise(A, p, s, G)
    bad = A.copy()
    bad[0, 17] = np.nan
    if M > 1:
        bad[M - 1, 900] = np.inf
    got = host(lb.gemm_w4a16_groupwise(dev(bad), dev(p), dev(s), G))
    want = chk.gemm_w4a16_groupwise(bad, p, s, G)
    assert not np.isfinite(want[0]).any() and not np.isfinite(got[0]).any()
    if M > 1:
        assert not np.isfinite(got[M - 1]).any()
    if M > 2:
        assert_close(got[1:M - 1], clean[1:M - 1], what="rows without a fault")
    poll_ok()


def test_w4a16_linearity_and_determinism():
    K, N, G = 2048, 2048, 128
    g = torch.Generator(device="cuda").manual_seed(5)
    W = torch.randn(K, N, device="cuda", generator=g) * 0.02
    p, s = lb.q4_quantize_groupwise(W, G)
    a = torch.randn(4, K, device="cuda", generator=g)
    b = torch.randn(4, K, device="cuda", generator=g)
    ya, yb = lb.gemm_w4a16_groupwise(a, p, s, G), lb.gemm_w4a16_groupwise(b, p, s, G)
    yab = lb.gemm_w4a16_groupwise(a + b, p, s, G)
    assert_close(host(yab), host(ya + yb), what="linearity")
    assert torch.equal(ya, lb.gemm_w4a16_groupwise(a, p, s, G)), "run-to-run determinism"
    # against the dequantised weights in fp64
    ref = (a.double() @ lb.q4_dequantize_groupwise(p, s, G).double()).float()
    assert_close(host(ya), host(ref), what="dequant + fp64 matmul")
    poll_ok()


# --------------------------------------------------------------------------- W8A16

def test_w8a16_golden():
    g = gio.load("w8a16_m16n64k128")
    got = lb.gemm_w8a16_perchannel(dev(g["A"]), dev(g["Bq"]), dev(g["b_s"]))
    assert_close(host(got), g["C"], what="w8a16 golden")


@pytest.mark.parametrize("M,N,K", [(16, 4096, 4096), (1, 1040, 1024), (7, 33, 100), (40, 512, 768)])
def test_w8a16_against_checker(chk, lib, M, N, K):
    rng = np.random.default_rng(M * 7 + N + K)
    A = rng.standard_normal((M, K)).astype(np.float32)
    W = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    q, s = lb.q8_quantize_per_col(dev(W))
    q0, s0 = chk.q8_quantize_per_col(W)
    assert_same_bits(host(q), q0, "q"); assert_same_bits(host(s), s0, "s")
    got = lb.gemm_w8a16_perchannel(dev(A), q, s)
    assert_close(host(got), chk.gemm_w8a16_perchannel(A, q0, s0),
                 what=f"w8a16 {M}x{N}x{K} fast={lib.lhb_gemm_w8a16_fast_path(M, N, K)}")
    C0 = rng.standard_normal((M, N)).astype(np.float32)
    got = lb.gemm_w8a16_perchannel(dev(A), q, s, C=dev(C0), alpha=0.5, beta=2.0)
    assert_close(host(got), chk.gemm_w8a16_perchannel(A, q0, s0, C0, alpha=0.5, beta=2.0), what="alpha/beta")
    poll_ok()


# --------------------------------------------------------------------------- append

def test_append_q8_golden_bits():
    g = gio.load("append_q8")
    L = Layout(*[int(v) for v in g["layout"]])
    shp = (L.num_blocks, L.n_kv_heads, L.block_size, L.head_dim)
    k = torch.zeros(shp, dtype=torch.int8, device="cuda"); v = torch.zeros_like(k)
    ks = torch.zeros(shp[:3], device="cuda"); vs = torch.zeros_like(ks)
    table = dev(g["table"])
    kn, vn = g["k_new"], g["v_new"]
    lb.paged_kv_append_q8(k, v, ks, vs, dev(kn[:, :5]), dev(vn[:, :5]), table, lb_layout(L), 0, 5)
    lb.paged_kv_append_q8(k, v, ks, vs, dev(kn[:, 5:]), dev(vn[:, 5:]), table, lb_layout(L), 5, 4)
    assert_same_bits(host(k), g["k"], "k pool"); assert_same_bits(host(v), g["v"], "v pool")
    assert_same_bits(host(ks), g["ks"], "k scales"); assert_same_bits(host(vs), g["vs"], "v scales")


# --------------------------------------------------------------------------- attention

@pytest.mark.parametrize("name", gio.names("attn_"))
def test_attention_golden(name, lib):
    g = gio.load(name)
    L, cfg = gio.attn_structs(g)
    got = lb.paged_attention_q8_batched(dev(g["Q"]), dev(g["k"]), dev(g["v"]), dev(g["ks"]),
                                        dev(g["vs"]), dev(g["tables"]), dev(g["seq_lens"]),
                                        lb_cfg(cfg), lb_layout(L))
    fast = lib.lhb_paged_attention_q8_fast_path(C.byref(lb_cfg(cfg)), C.byref(lb_layout(L)))
    assert_close(host(got), g["O"], what=f"{name} (fast={fast})")
    # single-request entry point, request by request
    for r in range(g["Q"].shape[0]):
        o = lb.paged_attention_q8(dev(g["Q"][r]), dev(g["k"]), dev(g["v"]), dev(g["ks"]), dev(g["vs"]),
                                  dev(g["tables"][r]), int(g["seq_lens"][r]), lb_cfg(cfg), lb_layout(L))
        assert_close(host(o), g["O"][r], what=f"{name} request {r}")
    gotf = lb.paged_attention_batched_f32(dev(g["Q"]), dev(g["kf"]), dev(g["vf"]), dev(g["tables"]),
                                          dev(g["seq_lens"]), lb_cfg(cfg), lb_layout(L))
    assert_close(host(gotf), g["O_f32"], what=name + " fp32 pools")
    poll_ok()


def build_paged_case(chk, rng, n_req, lens, qh, kvh, d, bs, nblk, batched_append=True):
    """Fill int8 pools on the GPU (library append) and on the CPU (checker) from the same rows."""
    L = Layout(nblk, bs, kvh, d)
    max_blocks = max(1, max((l + bs - 1) // bs for l in lens))
    perm = rng.permutation(nblk).astype(np.int32)
    tables = np.full((n_req, max_blocks), -1, np.int32)
    used = 0
    for r, l in enumerate(lens):
        nb = (l + bs - 1) // bs
        tables[r, :nb] = perm[used:used + nb]; used += nb
    assert used <= nblk
    pools = chk.empty_pools_q8(L)
    shp = (nblk, kvh, bs, d)
    k = torch.zeros(shp, dtype=torch.int8, device="cuda"); v = torch.zeros_like(k)
    ks = torch.zeros(shp[:3], device="cuda"); vs = torch.zeros_like(ks)
    tables_d = dev(tables)
    offs, kn_all, vn_all = [], [], []
    off = 0
    for r, l in enumerate(lens):
        kn = rng.standard_normal((kvh, l, d)).astype(np.float32)
        vn = rng.standard_normal((kvh, l, d)).astype(np.float32)
        offs.append(off); off += kn.size
        kn_all.append(kn.ravel()); vn_all.append(vn.ravel())
        if l:
            lb.paged_kv_append_q8(k, v, ks, vs, dev(kn), dev(vn), tables_d[r], lb_layout(L), 0, l)
    kn_all = np.concatenate(kn_all) if off else np.zeros(1, np.float32)
    vn_all = np.concatenate(vn_all) if off else np.zeros(1, np.float32)
    chk.paged_kv_append_q8_batched(pools, kn_all, vn_all, np.array(offs, np.int64), tables,
                                   np.zeros(n_req, np.int32), np.array(lens, np.int32), L)
    return L, tables, pools, (k, v, ks, vs)


@pytest.mark.parametrize("lens", [[513, 16, 1, 257, 4096, 33], [100] * 8, [0, 5, 0]])
def test_decode_attention_against_checker(chk, lib, lens):
    rng = np.random.default_rng(sum(lens) + len(lens))
    qh, kvh, d, bs = 32, 8, 128, 16
    nblk = sum((l + bs - 1) // bs for l in lens) + 7
    L, tables, pools, (k, v, ks, vs) = build_paged_case(chk, rng, len(lens), lens, qh, kvh, d, bs, nblk)
    assert_same_bits(host(k), pools.k, "k pool"); assert_same_bits(host(vs), pools.vs, "v scales")
    cfg = AttnCfg(qh, kvh, 1, d, 1, 0.0, 0, 0)
    Q = rng.standard_normal((len(lens), qh, 1, d)).astype(np.float32)
    sl = np.array(lens, np.int32)
    want = chk.paged_attention_q8_batched(Q, pools, tables, sl, cfg, L, parallel=True)
    got = lb.paged_attention_q8_batched(dev(Q), k, v, ks, vs, dev(tables), dev(sl), lb_cfg(cfg), lb_layout(L))
    fast = lib.lhb_paged_attention_q8_fast_path(C.byref(lb_cfg(cfg)), C.byref(lb_layout(L)))
    assert_close(host(got), want, what=f"decode lens={lens} fast={fast}")
    poll_ok()


def test_decode_step_append_then_attend(chk):
    """One decode step for a batch: batched append of one token per request at
    positions taken from the device seq_lens, then attention over len+1 keys."""
    rng = np.random.default_rng(77)
    qh, kvh, d, bs = 8, 2, 128, 16
    lens = [31, 16, 47, 1]
    nblk = 24
    L, tables, pools, (k, v, ks, vs) = build_paged_case(chk, rng, len(lens), [l + 1 for l in lens], qh, kvh, d, bs, nblk)
    # overwrite the last token of every request through the batched append
    kn = rng.standard_normal((len(lens), kvh, 1, d)).astype(np.float32)
    vn = rng.standard_normal((len(lens), kvh, 1, d)).astype(np.float32)
    past = np.array(lens, np.int32)
    lb.paged_kv_append_q8_batched(k, v, ks, vs, dev(kn), dev(vn), dev(tables), dev(past), lb_layout(L), 1)
    for r, l in enumerate(lens):
        chk.paged_kv_append_q8(pools, kn[r].copy(), vn[r].copy(), tables[r], L, l, 1)
    assert_same_bits(host(k), pools.k, "k after decode append"); assert_same_bits(host(ks), pools.ks, "ks")
    cfg = AttnCfg(qh, kvh, 1, d, 1, 0.0, 0, 0)
    Q = rng.standard_normal((len(lens), qh, 1, d)).astype(np.float32)
    sl = past + 1
    want = chk.paged_attention_q8_batched(Q, pools, tables, sl, cfg, L)
    got = lb.paged_attention_q8_batched(dev(Q), k, v, ks, vs, dev(tables), dev(sl), lb_cfg(cfg), lb_layout(L))
    assert_close(host(got), want, what="decode step")
    poll_ok()


def test_attention_ignores_table_padding_and_is_deterministic(chk):
    rng = np.random.default_rng(3)
    lens = [300, 40]
    L, tables, pools, (k, v, ks, vs) = build_paged_case(chk, rng, 2, lens, 8, 2, 128, 16, 40)
    cfg = lb_cfg(AttnCfg(8, 2, 1, 128, 1, 0.0, 0, 0))
    Q = dev(rng.standard_normal((2, 8, 1, 128)).astype(np.float32))
    sl = dev(np.array(lens, np.int32))
    a = lb.paged_attention_q8_batched(Q, k, v, ks, vs, dev(tables), sl, cfg, lb_layout(L))
    t2 = tables.copy(); t2[t2 < 0] = 12345678      # padding must never be dereferenced
    wide = np.full((2, tables.shape[1] + 9), -1, np.int32); wide[:, :tables.shape[1]] = t2
    b = lb.paged_attention_q8_batched(Q, k, v, ks, vs, dev(wide), sl, cfg, lb_layout(L))
    # a wider table may change the KV split, i.e. the order of the fp32 sums, not the values
    assert_close(host(b), host(a), rtol=1e-4, atol=1e-5, what="padding")
    a2 = lb.paged_attention_q8_batched(Q, k, v, ks, vs, dev(tables), sl, cfg, lb_layout(L))
    assert torch.equal(a, a2), "run-to-run determinism"
    poll_ok()


@pytest.mark.parametrize("d", [16, 128])
def test_attention_masks_a_released_page_inside_the_sequence(chk, d):
    """A table entry of -1 (or any id outside the pool) inside seq_len - what the cache manager
    leaves behind for a released page - masks that page's keys instead of being dereferenced: the
    result equals softmax attention over the remaining keys.  head_dim 16 takes the generic kernel,
    128 the decode kernel."""
    rng = np.random.default_rng(11 + d)
    qh, kvh, bs, nblk = 4, 2, 16, 12
    lens = [70, 40]
    L, tables, pools, (k, v, ks, vs) = build_paged_case(chk, rng, 2, lens, qh, kvh, d, bs, nblk)
    holed = tables.copy()
    holed[0, 1] = -1                     # tokens 16..31 of request 0
    holed[1, 2] = nblk + 5               # tokens 32..39 of request 1: beyond the pool
    Q = rng.standard_normal((2, qh, 1, d)).astype(np.float32)
    cfg = AttnCfg(qh, kvh, 1, d, 1, 0.0, 0, 0)
    got = host(lb.paged_attention_q8_batched(dev(Q), k, v, ks, vs, dev(holed), dev(np.array(lens, np.int32)),
                                              lb_cfg(cfg), lb_layout(L)))
    kq, vq = pools.k.reshape(nblk, kvh, bs, d).astype(np.float64), pools.v.reshape(nblk, kvh, bs, d).astype(np.float64)
    ksc, vsc = pools.ks.reshape(nblk, kvh, bs).astype(np.float64), pools.vs.reshape(nblk, kvh, bs).astype(np.float64)
    want = np.zeros_like(got, dtype=np.float64)
    for r, l in enumerate(lens):
        for h in range(qh):
            kvh_i = h // (qh // kvh)
            keys = [j for j in range(l) if 0 <= holed[r, j // bs] < nblk]
            blk = np.array([holed[r, j // bs] for j in keys]); slot = np.array([j % bs for j in keys])
            kk = kq[blk, kvh_i, slot] * ksc[blk, kvh_i, slot][:, None]
            vv = vq[blk, kvh_i, slot] * vsc[blk, kvh_i, slot][:, None]
            s = kk @ Q[r, h, 0].astype(np.float64) / np.sqrt(d)
            w = np.exp(s - s.max()); w /= w.sum()
            want[r, h, 0] = w @ vv
    assert_close(got, want, what=f"masked pages d={d}")
    poll_ok()


def test_batched_append_outside_the_table_row_writes_nothing(chk):
    """A request whose position lies at or past max_blocks * block_size (or is negative) has no
    table entry: the append must not fall through to the next request's row and quantise into its
    page.  The other requests' rows are written as usual, bit for bit."""
    rng = np.random.default_rng(5)
    kvh, d, bs, nblk, max_blocks = 2, 128, 16, 8, 2
    L = Layout(nblk, bs, kvh, d)
    tables = np.array([[0, 1], [2, 3], [4, 5]], np.int32)
    past = np.array([max_blocks * bs, 5, -3], np.int32)          # request 0: one past its row; request 2: negative
    shp = (nblk, kvh, bs, d)
    k = torch.full(shp, 7, dtype=torch.int8, device="cuda"); v = torch.full(shp, 9, dtype=torch.int8, device="cuda")
    ks = torch.full(shp[:3], 0.5, device="cuda"); vs = torch.full(shp[:3], 0.25, device="cuda")
    kn = rng.standard_normal((3, kvh, 1, d)).astype(np.float32)
    vn = rng.standard_normal((3, kvh, 1, d)).astype(np.float32)
    lb.paged_kv_append_q8_batched(k, v, ks, vs, dev(kn), dev(vn), dev(tables), dev(past), lb_layout(L), 1)
    pools = chk.empty_pools_q8(L)
    pools.k[:] = 7; pools.v[:] = 9; pools.ks[:] = 0.5; pools.vs[:] = 0.25
    chk.paged_kv_append_q8(pools, kn[1].copy(), vn[1].copy(), tables[1], L, 5, 1)      # only request 1 has a place
    assert_same_bits(host(k).reshape(-1), pools.k.reshape(-1), "k pool")
    assert_same_bits(host(v).reshape(-1), pools.v.reshape(-1), "v pool")
    assert_same_bits(host(ks).reshape(-1), pools.ks.reshape(-1), "k scales")
    assert_same_bits(host(vs).reshape(-1), pools.vs.reshape(-1), "v scales")
    # the fused QKV + rotary + append form applies the same rule
    qh = 4
    qkv = rng.standard_normal((3, (qh + 2 * kvh) * d)).astype(np.float32)
    k2 = torch.full(shp, 7, dtype=torch.int8, device="cuda"); v2 = torch.full(shp, 9, dtype=torch.int8, device="cuda")
    ks2 = torch.full(shp[:3], 0.5, device="cuda"); vs2 = torch.full(shp[:3], 0.25, device="cuda")
    q_out = torch.empty(3, qh, d, device="cuda")
    lb.qkv_rope_append_q8_decode(dev(qkv), q_out, k2, v2, ks2, vs2, dev(tables), dev(past), qh, lb_layout(L),
                                 theta_base=500000.0, interleaved=False)
    touched = (host(k2) != 7).reshape(nblk, -1).any(axis=1)
    assert touched.tolist() == [False, False, True, False, False, False, False, False], touched
    poll_ok()


# --------------------------------------------------------------------------- cache manager on the device

def test_device_cache_manager_end_to_end(chk):
    """tests/test_cache_manager.cpp:96-141 of the reference with int8 pools:
    create request -> allocate -> append -> attend, all through the manager's
    device-resident tables."""
    rng = np.random.default_rng(1400)
    qh, kvh, d, bs = 4, 2, 128, 16
    L = lb.PagedLayout(32, bs, kvh, d)
    cm = lb.DeviceCacheManager(L, max_requests=4, max_blocks_per_req=8)
    lens = [45, 7, 100]
    ids = [cm.create_request() for _ in lens]
    for rid, l in zip(ids, lens):
        assert cm.ensure_capacity(rid, l + 1)
        cm.set_seq_len(rid, l)
    assert not cm.ensure_capacity(ids[0], 8 * bs + 1)       # beyond max_blocks_per_req
    k, v, ks, vs, tables, seq_lens = cm.tensors()
    cl = Layout(32, bs, kvh, d)
    pools = chk.empty_pools_q8(cl)
    htab = np.full((4, 8), -1, np.int32)
    for rid, l in zip(ids, lens):
        htab[rid, :len(cm.block_table(rid))] = cm.block_table(rid)
        kn = rng.standard_normal((kvh, l, d)).astype(np.float32)
        vn = rng.standard_normal((kvh, l, d)).astype(np.float32)
        lb.paged_kv_append_q8(k, v, ks, vs, dev(kn), dev(vn), tables[rid], L, 0, l)
        chk.paged_kv_append_q8(pools, kn, vn, htab[rid], cl, 0, l)
    assert np.array_equal(host(tables), htab)
    assert host(seq_lens).tolist() == [45, 7, 100, 0]
    Q = rng.standard_normal((4, qh, 1, d)).astype(np.float32)
    cfg = AttnCfg(qh, kvh, 1, d, 1, 0.0, 0, 0)
    got = lb.paged_attention_q8_batched(dev(Q), k, v, ks, vs, tables, seq_lens, lb_cfg(cfg), L)
    want = chk.paged_attention_q8_batched(Q, pools, htab, np.array([45, 7, 100, 0], np.int32), cfg, cl)
    assert_close(host(got), want, what="managed blocks")
    cm.release_request(ids[1])
    torch.cuda.synchronize()
    assert (host(tables)[ids[1]] == -1).all() and host(seq_lens)[ids[1]] == 0
    cm.close()


# --------------------------------------------------------------------------- decode-step glue

@pytest.mark.parametrize("name", gio.names("rmsnorm_"))
def test_rmsnorm_golden(name):
    g = gio.load(name)
    y = lb.rmsnorm(dev(g["x"]), dev(g["gamma"]), float(g["eps"]))
    assert_close(host(y), g["y"], what=name)


@pytest.mark.parametrize("rows,dim", [(1, 4096), (32, 4096), (7, 14336), (3, 1001)])
def test_rmsnorm_against_checker(chk, rows, dim):
    rng = np.random.default_rng(rows + dim)
    x = (rng.standard_normal((rows, dim)) * rng.choice([1e-2, 1.0, 50.0])).astype(np.float32)
    gamma = rng.uniform(0.5, 1.5, dim).astype(np.float32)
    assert_close(host(lb.rmsnorm(dev(x), dev(gamma), 1e-5)), chk.rmsnorm(x, gamma, 1e-5), what=f"rmsnorm {rows}x{dim}")


@pytest.mark.parametrize("name", gio.names("rope_"))
def test_rope_golden(name):
    g = gio.load(name)
    y = lb.rope(dev(g["x"]), float(g["theta"]), float(g["freq_scale"]), bool(g["interleaved"]), int(g["pos_offset"]))
    assert_close(host(y), g["y"], what=name)


@pytest.mark.parametrize("interleaved", [True, False])
def test_rope_decode_batch_equals_per_request_calls(chk, interleaved):
    """One token per request at its own position = the reference called once per request with
    seq = 1 and pos_offset = that position (Llama-3 sizes: 32 + 8 heads of 128, theta 500000)."""
    rng = np.random.default_rng(17)
    n_req, n_heads, hd = 9, 40, 128
    x = rng.standard_normal((n_req, n_heads, hd)).astype(np.float32)
    pos = rng.integers(0, 8192, n_req).astype(np.int32)
    want = np.stack([chk.rope(x[r:r + 1], 500000.0, 1.0, interleaved, int(pos[r]))[0] for r in range(n_req)])
    got = lb.rope_decode_batched(dev(x), dev(pos), 500000.0, 1.0, interleaved)
    assert_close(host(got), want, what="rope decode batch")


@pytest.mark.parametrize("name", gio.names("swiglu_"))
def test_swiglu_golden(name):
    g = gio.load(name)
    assert_close(host(lb.swiglu(dev(g["x"]))), g["y"], what=name)


@pytest.mark.parametrize("rows,dim", [(1, 14336), (32, 14336), (5, 1003)])
def test_swiglu_against_checker(chk, rows, dim):
    rng = np.random.default_rng(rows * 3 + dim)
    x = (rng.standard_normal((rows, 2 * dim)) * 3).astype(np.float32)
    assert_close(host(lb.swiglu(dev(x))), chk.swiglu(x), what=f"swiglu {rows}x{dim}")


# --------------------------------------------------------------------------- asymmetric int4

@pytest.mark.parametrize("name", gio.names("q4a_"))
def test_q4a_golden_bits_and_gemm(name):
    g = gio.load(name)
    G = int(g["G"])
    p, s, z = lb.q4a_quantize_groupwise(dev(g["w"]), G)
    assert_same_bits(host(p), g["p"], "packed")
    assert_same_bits(host(s).view(np.uint16), g["s"], "scales")
    assert_same_bits(host(z).view(np.uint16), g["z"], "zero-points")
    assert_same_bits(host(lb.q4a_dequantize_groupwise(p, s, z, G)), g["d"], "dequant")
    assert_close(host(lb.gemm_w4a16_asym(dev(g["A"]), p, s, z, G)), g["C"], what=name)
    got = lb.gemm_w4a16_asym(dev(g["A"]), p, s, z, G, C=dev(g["C0"]), alpha=0.5, beta=2.0)
    assert_close(host(got), g["C_ab"], what=name + " alpha/beta")
    poll_ok()


@pytest.mark.parametrize("M", [1, 2, 8, 16, 32])
@pytest.mark.parametrize("N,K,G", [(1040, 1024, 128), (14336, 4096, 128), (256, 384, 64)])
def test_w4a16_asym_against_checker(lib, M, N, K, G):
    from cpu_checker import Checker
    chk = Checker("lho")            # the scheme is an extension: only the C statement of its rules has it
    rng = np.random.default_rng(7000 + M + N + K)
    A = chk.round_to_bf16((rng.standard_normal((M, K)) * rng.choice([1e-2, 1.0])).astype(np.float32))
    W = (rng.standard_normal((K, N)) * 0.02 + 0.01).astype(np.float32)
    p0, s0, z0 = chk.q4a_quantize_groupwise(W, G)
    p, s, z = lb.q4a_quantize_groupwise(dev(W), G)
    assert_same_bits(host(p), p0, "packed"); assert_same_bits(host(s).view(np.uint16), s0.view(np.uint16), "scales")
    assert_same_bits(host(z).view(np.uint16), z0.view(np.uint16), "zero-points")
    want = chk.gemm_w4a16_asym(A, p0, s0, z0, G)
    got = lb.gemm_w4a16_asym(dev(A), p, s, z, G)
    assert_close(host(got), want,
                 what=f"w4a16 asym M={M} N={N} K={K} G={G} fast={lib.lhb_gemm_w4a16_asym_fast_path(M, N, K, G)}")
    # activations a hundred times larger: the CPU loop's own fp32 rounding (partial sums of ~1e2) is then
    # above 1e-4, so the yardstick is the fp64 product with the dequantised weights, absolute bound scaled
    A100 = (A * 100.0).astype(np.float32)
    d = chk.q4a_dequantize_groupwise(p0, s0, z0, G).astype(np.float64)
    assert_close(host(lb.gemm_w4a16_asym(dev(A100), p, s, z, G)), A100.astype(np.float64) @ d, atol=1e-2,
                 what="w4a16 asym, activations x100, vs fp64")
    poll_ok()


# --------------------------------------------------------------------------- scheduler on the device tables

def test_scheduler_device_view_matches_reference_trace():
    """Device-backed scheduler: the dense block tables and seq_lens gathered on the GPU for every step equal
    the view the reference's Scheduler built on the host (recorded trace), padded to the fixed table width."""
    import json
    import os
    from test_cabi_cpu import _replay_scheduler
    trace = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "scheduler_trace.json")))
    L = lb.PagedLayout(trace["num_blocks"], trace["block_size"], 2, 8)
    mgr = lb.DeviceCacheManager(L, max_requests=64, max_blocks_per_req=8)
    sched = lb.DeviceScheduler(mgr, trace["max_concurrent"])

    def check_step(step, want):
        n, mb = len(want["ids"]), step.max_blocks_per_req
        torch.cuda.synchronize()
        tab = host(step.block_tables)
        assert tab.shape == (n, mb)
        ref = np.full((n, mb), -1, np.int32)
        ref[:, :want["max_blocks"]] = np.asarray(want["tables"], np.int32).reshape(n, want["max_blocks"])
        assert np.array_equal(tab, ref)
        assert host(step.seq_lens).tolist() == want["seq_lens"]
    _replay_scheduler(trace, mgr, sched, check_step)
    sched.close()
    mgr.close()
    poll_ok()


# --------------------------------------------------------------------------- FP8 E4M3

def test_fp8_quantisers_bit_exact():
    g = gio.load("fp8_quant")
    x = dev(g["x"])
    qt, st = lb.fp8_quantize_per_tensor(x)
    assert_same_bits(host(qt), g["qt"], "per tensor"); assert host(st)[0] == g["st"]
    qr, sr = lb.fp8_quantize_per_row(x)
    assert_same_bits(host(qr), g["qr"], "per row"); assert_same_bits(host(sr), g["sr"], "row scales")
    qc, sc = lb.fp8_quantize_per_col(x)
    assert_same_bits(host(qc), g["qc"], "per col"); assert_same_bits(host(sc), g["sc"], "col scales")
    assert_same_bits(host(lb.fp8_dequantize(qt, st, 0)), g["dt"], "dequant tensor")
    assert_same_bits(host(lb.fp8_dequantize(qr, sr, 1)), g["dr"], "dequant row")
    assert_same_bits(host(lb.fp8_dequantize(qc, sc, 2)), g["dc"], "dequant col")
    # every conversion case of the fixture, through the per-tensor quantiser with scale 1 (max = 448)
    c = gio.load("fp8_convert")
    keep = np.isfinite(c["x"]) & (np.abs(c["x"]) <= 448.0)
    v = np.concatenate([c["x"][keep], np.array([448.0], np.float32)])
    q, s = lb.fp8_quantize_per_tensor(dev(v))
    assert host(s)[0] == 1.0
    assert_same_bits(host(q)[:-1], c["bits"][keep], "conversion cases")
    poll_ok()


@pytest.mark.parametrize("name", gio.names("fp8_gemm_"))
def test_fp8_gemm_golden(name):
    g = gio.load(name)
    got = lb.gemm_fp8_e4m3(dev(g["A"]), dev(g["B"]), float(g["sa"]), float(g["sb"]))
    assert_close(host(got), g["C"], what=name)
    got = lb.gemm_fp8_e4m3(dev(g["A"]), dev(g["B"]), float(g["sa"]), float(g["sb"]), C=dev(g["C0"]), alpha=0.5, beta=2.0)
    assert_close(host(got), g["C_ab"], what=name + " alpha/beta")
    poll_ok()


@pytest.mark.parametrize("M,N,K", [(128, 256, 512), (300, 1040, 768), (1024, 2048, 1024)])
def test_fp8_gemm_tensor_core_path_against_checker(chk, lib, M, N, K):
    """Shapes served by tcgen05 (kind::f8f6f4), single-CTA and CTA-pair tiles, against the reference loop."""
    assert lib.lhb_gemm_fp8_fast_path(M, N, K) == 1
    rng = np.random.default_rng(M + N + K)
    A, sa = chk.fp8_quantize_per_tensor(rng.standard_normal((M, K)).astype(np.float32))
    B, sb = chk.fp8_quantize_per_tensor((rng.standard_normal((K, N)) * 0.02).astype(np.float32))
    C0 = rng.standard_normal((M, N)).astype(np.float32)
    want = chk.gemm_fp8_e4m3(A, B, sa, sb, C0, alpha=0.75, beta=1.0)
    got = lb.gemm_fp8_e4m3(dev(A), dev(B), sa, sb, C=dev(C0), alpha=0.75, beta=1.0)
    assert_close(host(got), want, what=f"fp8 gemm {M}x{N}x{K}")
    poll_ok()


def test_fused_qkv_rope_append_equals_the_three_calls():
    """lhb_qkv_rope_append_q8_decode = rope(q) + rope(k) + paged_kv_append_q8_batched, bit for bit."""
    rng = np.random.default_rng(91)
    n_req, hq, hkv, hd, bs, nb, mb = 6, 8, 2, 128, 16, 40, 6
    L = lb.PagedLayout(nb, bs, hkv, hd)
    pos = np.array([0, 5, 15, 16, 47, 80], np.int32)
    perm = rng.permutation(nb).astype(np.int32)
    tables = perm[:n_req * mb].reshape(n_req, mb).copy()
    qkv = dev(rng.standard_normal((n_req, (hq + 2 * hkv) * hd)).astype(np.float32))

    def pools():
        shape = (nb, hkv, bs, hd)
        return (torch.zeros(shape, dtype=torch.int8, device="cuda"), torch.zeros(shape, dtype=torch.int8, device="cuda"),
                torch.zeros(shape[:3], device="cuda"), torch.zeros(shape[:3], device="cuda"))
    for interleaved in (False, True):
        k1, v1, ks1, vs1 = pools()
        q1 = torch.empty(n_req, hq, hd, device="cuda")
        lb.qkv_rope_append_q8_decode(qkv, q1, k1, v1, ks1, vs1, dev(tables), dev(pos), hq, L, 500000.0, 1.0, interleaved)
        k2, v2, ks2, vs2 = pools()
        q2 = qkv[:, :hq * hd].contiguous().view(n_req, hq, hd)
        kk = qkv[:, hq * hd:(hq + hkv) * hd].contiguous().view(n_req, hkv, hd)
        vv = qkv[:, (hq + hkv) * hd:].contiguous().view(n_req, hkv, hd)
        lb.rope_decode_batched(q2, dev(pos), 500000.0, 1.0, interleaved)
        lb.rope_decode_batched(kk, dev(pos), 500000.0, 1.0, interleaved)
        lb.paged_kv_append_q8_batched(k2, v2, ks2, vs2, kk, vv, dev(tables), dev(pos), L, 1)
        assert torch.equal(q1, q2) and torch.equal(k1, k2) and torch.equal(v1, v2)
        assert torch.equal(ks1, ks2) and torch.equal(vs1, vs2)
    poll_ok()


@pytest.mark.parametrize("M", [1, 2, 3, 16, 18, 32, 40])
def test_w4a16_with_rmsnorm_and_swiglu_prologue(chk, lib, M):
    """RMSNorm / SwiGLU applied inside the GEMM's digit pass (or, for slabs of one or two rows, as
    separate launches by the wrapper) against the CPU composition of the two reference functions."""
    rng = np.random.default_rng(300 + M)
    K, N, G = 1024, 1040, 128
    W = (rng.standard_normal((K, N)) * 0.03).astype(np.float32)
    p, s = chk.q4_quantize_groupwise(W, G)
    dp, dsc = dev(p), dev(s)
    x = (rng.standard_normal((M, K)) * 3).astype(np.float32)
    gamma = rng.uniform(0.5, 1.5, K).astype(np.float32)
    C0 = rng.standard_normal((M, N)).astype(np.float32)
    want = chk.gemm_w4a16_groupwise(chk.rmsnorm(x, gamma, 1e-5), p, s, G, C0, alpha=1.0, beta=1.0)
    got = lb.gemm_w4a16_norm(dev(x), dev(gamma), 1e-5, dp, dsc, G, C=dev(C0), alpha=1.0, beta=1.0)
    assert_close(host(got), want, what=f"rmsnorm prologue M={M}")
    gu = (rng.standard_normal((M, 2 * K)) * 2).astype(np.float32)
    want = chk.gemm_w4a16_groupwise(chk.swiglu(gu), p, s, G)
    got = lb.gemm_w4a16_swiglu(dev(gu), dp, dsc, G)
    assert_close(host(got), want, what=f"swiglu prologue M={M}")
    poll_ok()

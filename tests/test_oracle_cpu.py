"""CPU suite: the C restatement against the golden fixtures (produced by the
reference's own compiled code) and, where the compiled reference is present,
against it directly on larger seeded inputs.  Integer outputs and scales must
be bit-identical; float outputs are bit-identical too because the restatement
keeps the reference's accumulation order."""
import numpy as np
import pytest

import golden_io as gio
from cpu_checker import AttnCfg, Checker, Layout, PagedPools, ref_available

port = Checker("lho")


def same(a, b):
    assert a.shape == b.shape and a.dtype == b.dtype
    assert np.array_equal(a.view(np.uint8), b.view(np.uint8))


def test_bf16_rounding_matches_reference_bits():
    g = gio.load("bf16_round")
    same(port.round_to_bf16(g["x"]), g["y"])


def test_q8_per_row_golden():
    g = gio.load("q8_per_row")
    q, s = port.q8_quantize_per_row(g["x"])
    same(q, g["q"]); same(s, g["s"])
    same(port.q8_dequantize_per_row(q, s), g["d"])
    assert s[3] == 1.0 and not q[3].any()          # zero row keeps scale 1
    assert np.abs(q).max() <= 127
    # reference invariant (tests/test_quant.cpp:24-47): |dq - x| < scale
    assert np.all(np.abs(g["d"] - g["x"]) < s[:, None] + 1e-6)


def test_q8_per_col_golden():
    g = gio.load("q8_per_col")
    q, s = port.q8_quantize_per_col(g["x"])
    same(q, g["q"]); same(s, g["s"])
    same(port.q8_dequantize_per_col(q, s), g["d"])
    assert s[5] == 1.0


@pytest.mark.parametrize("name", gio.names("q4_"))
def test_q4_groupwise_golden(name):
    g = gio.load(name)
    G = int(g["G"])
    p, s = port.q4_quantize_groupwise(g["w"], G)
    same(p, g["p"]); same(s, g["s"])
    same(port.q4_dequantize_groupwise(p, s, G), g["d"])
    K, N = g["w"].shape
    vals = np.array([[port.q4_get(p, k, n) for n in range(N)] for k in range(K)])
    assert vals.min() >= -7 and vals.max() <= 7     # tests/test_quant.cpp:85-99
    assert np.all(np.abs(g["d"] - g["w"]) < np.repeat(s, G, axis=0) + 1e-6)


def test_w8a8_golden():
    g = gio.load("w8a8_m32n48k64")
    C = port.gemm_w8a8(g["Aq"], g["Bq"], g["a_s"], g["b_s"])
    same(C, g["C"])
    rel = np.sqrt(np.mean((C - g["C_fp32"]) ** 2)) / np.sqrt(np.mean(g["C_fp32"] ** 2))
    assert rel < 0.05                                # tests/test_gemm_quant.cpp:31-53
    g = gio.load("w8a8_beta")
    same(port.gemm_w8a8(g["Aq"], g["Bq"], g["a_s"], g["b_s"], g["C0"], alpha=0.5, beta=2.0), g["C"])


@pytest.mark.parametrize("name", gio.names("w4a16_"))
def test_w4a16_golden(name):
    g = gio.load(name)
    G = int(g["G"])
    same(port.gemm_w4a16_groupwise(g["A"], g["p"], g["s"], G), g["C"])
    same(port.gemm_w4a16_groupwise(g["A"], g["p"], g["s"], G, g["C0"], alpha=0.5, beta=2.0), g["C_ab"])


def test_w8a16_golden():
    g = gio.load("w8a16_m16n64k128")
    same(port.gemm_w8a16_perchannel(g["A"], g["Bq"], g["b_s"]), g["C"])


def test_w4a16_packed_bytes_beat_fp16_by_3x():
    # tests/test_gemm_quant.cpp:126-138
    K = N = 4096
    for G in (32, 64, 128):
        assert (K * N * 2) / (K * N // 2 + K // G * N * 4) > 3.0


def test_append_q8_golden():
    g = gio.load("append_q8")
    L = Layout(*[int(v) for v in g["layout"]])
    pools = port.empty_pools_q8(L)
    kn, vn = g["k_new"], g["v_new"]
    port.paged_kv_append_q8(pools, kn[:, :5].copy(), vn[:, :5].copy(), g["table"], L, 0, 5)
    port.paged_kv_append_q8(pools, kn[:, 5:].copy(), vn[:, 5:].copy(), g["table"], L, 5, 4)
    same(pools.k, g["k"]); same(pools.v, g["v"]); same(pools.ks, g["ks"]); same(pools.vs, g["vs"])


@pytest.mark.parametrize("name", gio.names("attn_"))
def test_attention_golden(name):
    g = gio.load(name)
    L, cfg = gio.attn_structs(g)
    pools = PagedPools(g["k"], g["v"], g["ks"], g["vs"])
    O = port.paged_attention_q8_batched(g["Q"], pools, g["tables"], g["seq_lens"], cfg, L)
    same(O, g["O"])
    Of = port.paged_attention_f32_batched(g["Q"], g["kf"], g["vf"], g["tables"], g["seq_lens"], cfg, L)
    same(Of, g["O_f32"])
    # reference invariant (tests/test_kvcache_quant.cpp:71-127): q8 close to fp32
    assert np.mean((O - Of) ** 2) < 1e-3 and np.abs(O - Of).max() < 5e-2


@pytest.mark.skipif(not ref_available(), reason="compiled reference not present")
@pytest.mark.parametrize("name", gio.names("rmsnorm_"))
def test_rmsnorm_golden(name):
    g = gio.load(name)
    y = port.rmsnorm(g["x"], g["gamma"], float(g["eps"]))
    same(y, g["y"])
    # invariant of the reference's own test: unit gamma gives rows of RMS one
    u = port.rmsnorm(g["x"], np.ones_like(g["gamma"]), 0.0)
    rms = np.sqrt((u.astype(np.float64) ** 2).mean(axis=1))
    nz = np.abs(g["x"]).max(axis=1) > 0
    assert np.allclose(rms[nz], 1.0, atol=1e-5)


@pytest.mark.parametrize("name", gio.names("rope_"))
def test_rope_golden(name):
    g = gio.load(name)
    args = (float(g["theta"]), float(g["freq_scale"]), bool(g["interleaved"]), int(g["pos_offset"]))
    y = port.rope(g["x"], *args)
    same(y, g["y"])
    # a rotation keeps every pair's norm; position 0 without offset is the identity
    assert np.allclose((y.astype(np.float64) ** 2).sum(-1), (g["x"].astype(np.float64) ** 2).sum(-1), rtol=1e-5)
    if int(g["pos_offset"]) == 0:
        assert np.array_equal(y[0], g["x"][0])
    # one token at position p equals row p of the sequence call
    seq = g["x"].shape[0]
    one = port.rope(g["x"][seq - 1:seq], args[0], args[1], args[2], args[3] + seq - 1)
    same(one[0], y[seq - 1])


@pytest.mark.parametrize("name", gio.names("swiglu_"))
def test_swiglu_golden(name):
    g = gio.load(name)
    same(port.swiglu(g["x"]), g["y"])


def test_f16_conversion_matches_reference_bits():
    g = gio.load("f16_round")
    assert np.array_equal(port.f32_to_f16_bits(g["x"]), g["bits"])


@pytest.mark.parametrize("name", gio.names("q4a_"))
def test_q4a_fixture_properties(name):
    """Asymmetric int4: the fixture reproduces, zero-points are integers in [0, 15], zero is exactly
    representable, the round trip is within half a step, and the GEMM equals A @ dequant."""
    g = gio.load(name)
    G = int(g["G"])
    p, s, z = port.q4a_quantize_groupwise(g["w"], G)
    same(p, g["p"]); same(s.view(np.uint16), g["s"]); same(z.view(np.uint16), g["z"])
    zf, sf = z.astype(np.float32), s.astype(np.float32)
    assert np.all(zf == np.round(zf)) and zf.min() >= 0 and zf.max() <= 15
    d = port.q4a_dequantize_groupwise(p, s, z, G)
    same(d, g["d"])
    step = np.repeat(sf, G, axis=0)
    assert np.all(np.abs(g["w"] - d) <= 0.5 * step * (1 + 1e-3) + 1e-12)
    assert np.all(d[g["w"] == 0.0] == 0.0)
    same(port.gemm_w4a16_asym(g["A"], p, s, z, G), g["C"])
    same(port.gemm_w4a16_asym(g["A"], p, s, z, G, g["C0"], alpha=0.5, beta=2.0), g["C_ab"])
    ref = g["A"].astype(np.float64) @ d.astype(np.float64)
    assert np.allclose(g["C"], ref, rtol=1e-4, atol=1e-5)


def test_fp8_conversion_and_quantisers_golden():
    g = gio.load("fp8_convert")
    assert np.array_equal(port.f32_to_e4m3_bits(g["x"]), g["bits"])
    back = port.e4m3_bits_to_f32(np.arange(256, dtype=np.uint8))
    assert np.array_equal(back.view(np.uint32), g["back"].view(np.uint32))
    assert np.nanmax(np.abs(back)) == 448.0 and np.isnan(back[0x7f]) and np.isnan(back[0xff])
    g = gio.load("fp8_quant")
    qt, st = port.fp8_quantize_per_tensor(g["x"]); same(qt, g["qt"]); assert np.float32(st) == g["st"]
    qr, sr = port.fp8_quantize_per_row(g["x"]); same(qr, g["qr"]); same(sr, g["sr"])
    qc, sc = port.fp8_quantize_per_col(g["x"]); same(qc, g["qc"]); same(sc, g["sc"])
    same(port.fp8_dequantize(qt, [st], 0), g["dt"]); same(port.fp8_dequantize(qr, sr, 1), g["dr"])
    same(port.fp8_dequantize(qc, sc, 2), g["dc"])
    # the reference's own bound: a round trip is within 2^-4 of the magnitude (3 mantissa bits) or of the step
    assert np.all(np.abs(g["dr"] - g["x"]) <= np.maximum(np.abs(g["x"]) * 2.0 ** -4, sr[:, None] * 2.0 ** -9) + 1e-12)


@pytest.mark.parametrize("name", gio.names("fp8_gemm_"))
def test_fp8_gemm_golden(name):
    g = gio.load(name)
    same(port.gemm_fp8_e4m3(g["A"], g["B"], float(g["sa"]), float(g["sb"])), g["C"])
    same(port.gemm_fp8_e4m3(g["A"], g["B"], float(g["sa"]), float(g["sb"]), g["C0"], alpha=0.5, beta=2.0), g["C_ab"])


def test_port_matches_compiled_reference_on_larger_inputs():
    ref = Checker("lhr")
    rng = np.random.default_rng(7)
    # quantisers
    x = rng.standard_normal((37, 200)).astype(np.float32)
    for f in ("q8_quantize_per_row", "q8_quantize_per_col"):
        a, b = getattr(port, f)(x), getattr(ref, f)(x)
        same(a[0], b[0]); same(a[1], b[1])
    (qt, st), (qt2, st2) = port.q8_quantize_per_tensor(x), ref.q8_quantize_per_tensor(x)
    same(qt, qt2); same(st, st2)
    same(port.q8_dequantize_per_tensor(qt, st[0]), ref.q8_dequantize_per_tensor(qt, st[0]))
    zq, zs = port.q8_quantize_per_tensor(np.zeros(5, np.float32))
    assert float(zs[0]) == 1.0 and not zq.any()           # all-zero input: scale 1
    w = (rng.standard_normal((512, 96)) * 0.02).astype(np.float32)
    (p, s), (p2, s2) = port.q4_quantize_groupwise(w, 128), ref.q4_quantize_groupwise(w, 128)
    same(p, p2); same(s, s2)
    # GEMMs
    A = rng.standard_normal((3, 512)).astype(np.float32)
    same(port.gemm_w4a16_groupwise(A, p, s, 128), ref.gemm_w4a16_groupwise(A, p, s, 128))
    Bq, bs = ref.q8_quantize_per_col(w)
    same(port.gemm_w8a16_perchannel(A, Bq, bs), ref.gemm_w8a16_perchannel(A, Bq, bs))
    Aq, a_s = ref.q8_quantize_per_row(A)
    same(port.gemm_w8a8(Aq, Bq, a_s, bs), ref.gemm_w8a8(Aq, Bq, a_s, bs))
    # paged decode at the benchmark's geometry, small batch
    L = Layout(64, 16, 2, 128)
    cfg = AttnCfg(8, 2, 1, 128, 1, 0.0, 0, 0)
    lens = [200, 37, 129]
    tables = np.full((3, 13), -1, np.int32)
    perm = rng.permutation(64).astype(np.int32)
    pa, pb = port.empty_pools_q8(L), ref.empty_pools_q8(L)
    used = 0
    for r, l in enumerate(lens):
        nb = (l + 15) // 16
        tables[r, :nb] = perm[used:used + nb]; used += nb
        kn = rng.standard_normal((2, l, 128)).astype(np.float32)
        vn = rng.standard_normal((2, l, 128)).astype(np.float32)
        port.paged_kv_append_q8(pa, kn, vn, tables[r], L, 0, l)
        ref.paged_kv_append_q8(pb, kn, vn, tables[r], L, 0, l)
    same(pa.k, pb.k); same(pa.vs, pb.vs)
    Q = rng.standard_normal((3, 8, 1, 128)).astype(np.float32)
    sl = np.array(lens, np.int32)
    same(port.paged_attention_q8_batched(Q, pa, tables, sl, cfg, L),
         ref.paged_attention_q8_batched(Q, pb, tables, sl, cfg, L))
    same(port.paged_attention_q8_batched(Q, pa, tables, sl, cfg, L, parallel=True),
         ref.paged_attention_q8_batched(Q, pb, tables, sl, cfg, L))

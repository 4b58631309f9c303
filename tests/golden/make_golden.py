"""Regenerate tests/golden/*.npz from the reference's own compiled code.

Run where the reference checkout is present (it is compiled by
``make -C oracle ref`` into ``oracle/_ref/liblh_ref.so``):

    python tests/golden/make_golden.py

Each fixture stores the seeded inputs together with the outputs the reference
produced for them, so the fixtures are self-contained: the tests compare the C
restatement (CPU suite) and the CUDA path (GPU suite) with these outputs and
never need the reference checkout.  Shapes follow the reference's own unit
tests for this path (tests/test_quant.cpp, tests/test_gemm_quant.cpp,
tests/test_kvcache_quant.cpp, tests/test_paged_attention.cpp,
tests/test_cache_manager.cpp) plus a few edge cases (zero rows, exact ties,
saturation, ragged batches, permuted block tables, masks).
"""
from __future__ import annotations

import ctypes as C
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from cpu_checker import AttnCfg, Checker, Layout, ref_available  # noqa: E402


def save(name, **arrays):
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **arrays)
    print("wrote", name, {k: getattr(v, "shape", None) for k, v in arrays.items()})


def uniform(rng, shape, lo=-1.0, hi=1.0):
    return rng.uniform(lo, hi, size=shape).astype(np.float32)


def main():
    if not ref_available():
        raise SystemExit("oracle/_ref/liblh_ref.so missing: run `make -C oracle ref` first")
    ref = Checker("lhr")
    rng = np.random.default_rng(20240)

    # ---- bf16 rounding (ties, NaN, inf, subnormals) -----------------------
    x = np.concatenate([
        uniform(rng, 256, -4, 4),
        np.array([1.00390625, 1.01171875, -1.00390625, 3.0e-41, np.inf, -np.inf, 0.0, -0.0,
                  65504.0, 3.3895314e38], np.float32)])
    save("bf16_round", x=x, y=ref.round_to_bf16(x))

    # ---- q8 per row: magnitudes from 1e-2 to 1e2, a zero row, exact ties ---
    rows, dim = 8, 64
    x = uniform(rng, (rows, dim))
    x[0] *= 0.01
    x[7] *= 100.0
    x[3] = 0.0
    x[4, :] = np.round(x[4] * 8) / 8          # many values land on .5 after scaling
    x[4, 0] = 127.0 / 8                        # makes scale exactly 1/8
    q, s = ref.q8_quantize_per_row(x)
    save("q8_per_row", x=x, q=q, s=s, d=ref.q8_dequantize_per_row(q, s))

    # ---- q8 per col: a zero column, a huge column --------------------------
    x = uniform(rng, (16, 32))
    x[:, 5] = 0.0
    x[:, 9] *= 1e4
    q, s = ref.q8_quantize_per_col(x)
    save("q8_per_col", x=x, q=q, s=s, d=ref.q8_dequantize_per_col(q, s))

    # ---- q4 group-wise: the reference's test shape and a G=128 shape -------
    for tag, K, N, G in (("k64n16g32", 64, 16, 32), ("k256n48g128", 256, 48, 128),
                         ("k8n4g4", 8, 4, 4)):
        w = uniform(rng, (K, N)) * (0.02 if G == 128 else 1.0)
        if K >= 64:
            w[:G, 1] = 0.0                      # a zero group -> scale 1
        p, s = ref.q4_quantize_groupwise(w, G)
        save("q4_" + tag, w=w, G=np.int32(G), p=p, s=s, d=ref.q4_dequantize_groupwise(p, s, G))

    # ---- W8A8 GEMM (reference test shapes) ----------------------------------
    A, B = uniform(rng, (32, 64)), uniform(rng, (64, 48))
    Aq, a_s = ref.q8_quantize_per_row(A)
    Bq, b_s = ref.q8_quantize_per_col(B)
    save("w8a8_m32n48k64", Aq=Aq, Bq=Bq, a_s=a_s, b_s=b_s, C=ref.gemm_w8a8(Aq, Bq, a_s, b_s),
         C_fp32=ref.gemm_f32(A, B))
    A, B = uniform(rng, (4, 4)), uniform(rng, (4, 4))
    Aq, a_s = ref.q8_quantize_per_row(A)
    Bq, b_s = ref.q8_quantize_per_col(B)
    C0 = np.full((4, 4), 1.5, np.float32)
    save("w8a8_beta", Aq=Aq, Bq=Bq, a_s=a_s, b_s=b_s, C0=C0,
         C=ref.gemm_w8a8(Aq, Bq, a_s, b_s, C0, alpha=0.5, beta=2.0))

    # ---- W4A16 group-wise GEMM -------------------------------------------------
    for tag, M, N, K, G in (("m16n32k64g32", 16, 32, 64, 32), ("m1n256k512g128", 1, 256, 512, 128),
                            ("m8n144k256g128", 8, 144, 256, 128), ("m5n20k24g4", 5, 20, 24, 4)):
        A = uniform(rng, (M, K))
        W = uniform(rng, (K, N))
        p, s = ref.q4_quantize_groupwise(W, G)
        C0 = uniform(rng, (M, N))
        save("w4a16_" + tag, A=A, p=p, s=s, G=np.int32(G), C=ref.gemm_w4a16_groupwise(A, p, s, G),
             C0=C0, C_ab=ref.gemm_w4a16_groupwise(A, p, s, G, C0, alpha=0.5, beta=2.0))

    # ---- weight-only int8 per-channel GEMM (composition) -------------------------
    A = rng.standard_normal((16, 128)).astype(np.float32)
    W = (rng.standard_normal((128, 64)) * 0.02).astype(np.float32)
    Bq, b_s = ref.q8_quantize_per_col(W)
    save("w8a16_m16n64k128", A=A, Bq=Bq, b_s=b_s, C=ref.gemm_w8a16_perchannel(A, Bq, b_s))

    # ---- int8 append (reference test shape) + a second chunk ---------------------
    L = Layout(4, 4, 2, 8)
    S = 9
    kn, vn = uniform(rng, (2, S, 8)), uniform(rng, (2, S, 8))
    kn[1, 2] = 0.0                              # zero row -> scale 1
    table = np.array([2, 0, 3], np.int32)
    pools = ref.empty_pools_q8(L)
    ref.paged_kv_append_q8(pools, kn[:, :5].copy(), vn[:, :5].copy(), table, L, 0, 5)
    ref.paged_kv_append_q8(pools, kn[:, 5:].copy(), vn[:, 5:].copy(), table, L, 5, 4)
    save("append_q8", layout=np.array([4, 4, 2, 8], np.int32), k_new=kn, v_new=vn, table=table,
         k=pools.k, v=pools.v, ks=pools.ks, vs=pools.vs)

    # ---- int8 attention: single request (reference test shape) -------------------
    def attn_case(tag, qh, kvh, sq, lens, d, bs, nblk, causal=1, scale=0.0, window=0, chunk=0):
        L = Layout(nblk, bs, kvh, d)
        cfg = AttnCfg(qh, kvh, sq, d, causal, scale, window, chunk)
        n_req = len(lens)
        max_blocks = max((l + bs - 1) // bs for l in lens)
        perm = rng.permutation(nblk).astype(np.int32)
        tables = np.full((n_req, max_blocks), -1, np.int32)
        pools = ref.empty_pools_q8(L)
        kf = np.zeros((nblk, kvh, bs, d), np.float32)
        vf = np.zeros_like(kf)
        used = 0
        for r, l in enumerate(lens):
            nb = (l + bs - 1) // bs
            tables[r, :nb] = perm[used:used + nb]
            used += nb
            kn = rng.standard_normal((kvh, l, d)).astype(np.float32)
            vn = rng.standard_normal((kvh, l, d)).astype(np.float32)
            ref.paged_kv_append_q8(pools, kn, vn, tables[r], L, 0, l)
            ref.paged_kv_append_f32(kf, vf, kn, vn, tables[r], L, 0, l)
        Q = rng.standard_normal((n_req, qh, sq, d)).astype(np.float32)
        seq_lens = np.array(lens, np.int32)
        O = ref.paged_attention_q8_batched(Q, pools, tables, seq_lens, cfg, L)
        O1 = np.stack([ref.paged_attention_q8(Q[r], pools, tables[r], int(lens[r]), cfg, L)
                       for r in range(n_req)])
        assert np.array_equal(O, O1)
        Of = ref.paged_attention_f32_batched(Q, kf, vf, tables, seq_lens, cfg, L)
        save("attn_" + tag, layout=np.array([nblk, bs, kvh, d], np.int32),
             cfg_i=np.array([qh, kvh, sq, d, causal, window, chunk], np.int32),
             cfg_scale=np.float32(scale), Q=Q, k=pools.k, v=pools.v, ks=pools.ks, vs=pools.vs,
             kf=kf, vf=vf, tables=tables, seq_lens=seq_lens, O=O, O_f32=Of)

    attn_case("single_d16", 4, 2, 1, [32], 16, 8, 8)
    attn_case("ragged_d16", 4, 2, 1, [17, 9], 16, 4, 12)
    attn_case("decode_d128", 8, 2, 1, [70, 16, 1, 33], 128, 16, 16)
    attn_case("decode_d128_window", 8, 2, 1, [70, 40], 128, 16, 16, window=24)
    attn_case("decode_d128_chunk", 8, 2, 1, [70, 40], 128, 16, 16, chunk=32, scale=0.25)
    attn_case("prefill_d16", 4, 2, 5, [21, 6], 16, 4, 12)
    attn_case("prefill_d16_masks", 4, 2, 5, [21, 9], 16, 4, 12, window=7, chunk=8)
    attn_case("noncausal_d16", 2, 1, 3, [10], 16, 4, 4, causal=0)
    attn_case("empty_d16", 2, 1, 1, [0, 5], 16, 4, 4)

    # ---- cache manager allocation order --------------------------------------------
    L = Layout(8, 4, 2, 16)
    lib = ref.lib
    lib.lhr_cm_create.restype = C.c_void_p
    m = C.c_void_p(lib.lhr_cm_create(C.byref(L)))
    log = []

    def table(rid):
        buf = np.full(16, -7, np.int32)
        n = lib.lhr_cm_table(m, rid, buf.ctypes.data_as(C.c_void_p), 16)
        return buf[:n].tolist()

    r0 = lib.lhr_cm_create_request(m)
    ok = lib.lhr_cm_ensure_capacity(m, r0, 9)
    log.append(("r0", r0, ok, table(r0), lib.lhr_cm_num_free(m)))
    r1 = lib.lhr_cm_create_request(m)
    ok = lib.lhr_cm_ensure_capacity(m, r1, 13)
    log.append(("r1", r1, ok, table(r1), lib.lhr_cm_num_free(m)))
    ok = lib.lhr_cm_ensure_capacity(m, r1, 40)          # OOM: unchanged
    log.append(("r1_oom", r1, ok, table(r1), lib.lhr_cm_num_free(m)))
    lib.lhr_cm_release_request(m, r0)
    r2 = lib.lhr_cm_create_request(m)                   # id recycled
    ok = lib.lhr_cm_ensure_capacity(m, r2, 16)          # LIFO reuse of r0's blocks
    log.append(("r2", r2, ok, table(r2), lib.lhr_cm_num_free(m)))
    ok = lib.lhr_cm_reference_block(m, r2, 5, table(r1)[0])
    log.append(("r2_ref", r2, ok, table(r2), lib.lhr_cm_refcount(m, table(r1)[0])))
    lib.lhr_cm_destroy(m)
    import json
    with open(os.path.join(HERE, "cache_manager_trace.json"), "w") as f:
        json.dump(log, f)
    print("wrote cache_manager_trace", log)


def glue_fixtures():
    """RMSNorm / RoPE / SwiGLU (src/kernels/normalization.cpp, rope.cpp, activation.cpp); shapes
    follow tests/test_normalization.cpp, tests/test_rope.cpp and tests/test_activation.cpp plus
    the decode-step sizes (dim 4096, head_dim 128, theta 500000, position 2047)."""
    if not ref_available():
        raise SystemExit("oracle/_ref/liblh_ref.so missing: run `make -C oracle ref` first")
    ref = Checker("lhr")
    rng = np.random.default_rng(20244)
    x = uniform(rng, (5, 96), -3, 3)
    x[2] = 0.0                                   # zero row: y = 0, inv_rms = 1/sqrt(eps)
    x[3] *= 1e3
    g = uniform(rng, 96, 0.5, 1.5)
    save("rmsnorm_r5d96", x=x, gamma=g, eps=np.float32(1e-5), y=ref.rmsnorm(x, g, 1e-5))
    x = rng.standard_normal((3, 4096)).astype(np.float32)
    g = uniform(rng, 4096, 0.5, 1.5)
    save("rmsnorm_r3d4096", x=x, gamma=g, eps=np.float32(1e-6), y=ref.rmsnorm(x, g, 1e-6))
    for name, inter, theta, fs, off, shape in [
            ("rope_interleaved", True, 10000.0, 1.0, 0, (6, 2, 16)),
            ("rope_half_offset", False, 10000.0, 1.0, 37, (4, 3, 32)),
            ("rope_half_llama3", False, 500000.0, 1.0, 2047, (2, 8, 128)),
            ("rope_scaled", True, 10000.0, 0.25, 5, (3, 2, 64))]:
        x = rng.standard_normal(shape).astype(np.float32)
        save(name, x=x, theta=np.float32(theta), freq_scale=np.float32(fs), interleaved=np.int32(inter),
             pos_offset=np.int32(off), y=ref.rope(x, theta, fs, inter, off))
    x = (rng.standard_normal((4, 2 * 50)) * 4).astype(np.float32)
    x[0, :4] = [0.0, -30.0, 30.0, -100.0]        # sigmoid tails
    save("swiglu_r4d50", x=x, y=ref.swiglu(x))
    x = rng.standard_normal((2, 2 * 1024)).astype(np.float32)
    save("swiglu_r2d1024", x=x, y=ref.swiglu(x))


def asym_fixtures():
    """Asymmetric int4 (fp16 scale and zero-point per group).  The reference has no such scheme, so
    these vectors come from the C restatement of the rules written in include/lhb200.h (parity
    unpinned); only the fp16 conversion inside them is pinned, against lh::half, here."""
    port = Checker("lho")
    rng = np.random.default_rng(20246)
    if ref_available():
        ref = Checker("lhr")
        x = np.concatenate([rng.standard_normal(4096).astype(np.float32) *
                            rng.choice([1e-8, 1e-5, 1e-3, 1.0, 100.0, 70000.0], 4096).astype(np.float32),
                            np.array([0.0, -0.0, 65504.0, 65520.0, 6.1e-5, 5.96e-8, 2.98e-8, 1.0009765625,
                                      1.00048828125, 1.00146484375, np.inf, -np.inf], np.float32)])
        bits = ref.f32_to_f16_bits(x)
        assert np.array_equal(bits, port.f32_to_f16_bits(x))
        save("f16_round", x=x, bits=bits)
    for name, K, N, G, M in [("q4a_k256n48g128", 256, 48, 128, 3), ("q4a_k128n32g32", 128, 32, 32, 5),
                             ("q4a_k512n256g128", 512, 256, 128, 1)]:
        w = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
        w[: G, 1] = 0.0                          # an all-zero group: scale 1, zero-point 0
        w[:, 2] = np.abs(w[:, 2])                # one-sided groups: zero-point 0 / 15
        w[:, 3] = -np.abs(w[:, 3])
        p, s, z = port.q4a_quantize_groupwise(w, G)
        A = rng.standard_normal((M, K)).astype(np.float32)
        C0 = rng.standard_normal((M, N)).astype(np.float32)
        save(name, w=w, G=np.int32(G), p=p, s=s.view(np.uint16), z=z.view(np.uint16),
             d=port.q4a_dequantize_groupwise(p, s, z, G), A=A, C=port.gemm_w4a16_asym(A, p, s, z, G),
             C0=C0, C_ab=port.gemm_w4a16_asym(A, p, s, z, G, C0, alpha=0.5, beta=2.0))


def fp8_fixtures():
    """FP8 E4M3 (src/kernels/dtypes.hpp:111-196, quant.cpp:176-249, gemm_quant.cpp:87-104), shapes after
    tests/test_quant.cpp and tests/test_gemm_quant.cpp's fp8 cases, produced by the compiled reference."""
    if not ref_available():
        raise SystemExit("oracle/_ref/liblh_ref.so missing: run `make -C oracle ref` first")
    ref = Checker("lhr")
    rng = np.random.default_rng(20247)
    x = np.concatenate([rng.standard_normal(2048).astype(np.float32) *
                        rng.choice([1e-4, 1e-3, 1e-2, 0.1, 1.0, 30.0, 300.0, 1000.0], 2048).astype(np.float32),
                        np.array([0.0, -0.0, 448.0, 449.0, 464.0, 465.0, 480.0, 1e9, -1e9, np.inf, -np.inf, np.nan,
                                  2.0 ** -9, 2.0 ** -10, 2.0 ** -10 * 1.0001, 2.0 ** -11, 1.5 * 2.0 ** -9,
                                  0.0146484375, 0.9375, 0.96875, 1.0625], np.float32)])
    save("fp8_convert", x=x, bits=ref.f32_to_e4m3_bits(x), back=ref.e4m3_bits_to_f32(np.arange(256, dtype=np.uint8)))
    X = uniform(rng, (9, 80), -3, 3)
    X[2] = 0.0
    X[5] *= 100.0
    X[:, 7] = 0.0
    qt, st = ref.fp8_quantize_per_tensor(X)
    qr, sr = ref.fp8_quantize_per_row(X)
    qc, sc = ref.fp8_quantize_per_col(X)
    save("fp8_quant", x=X, qt=qt, st=np.float32(st), qr=qr, sr=sr, qc=qc, sc=sc,
         dt=ref.fp8_dequantize(qt, [st], 0), dr=ref.fp8_dequantize(qr, sr, 1), dc=ref.fp8_dequantize(qc, sc, 2))
    for name, M, N, K in [("fp8_gemm_m5n24k64", 5, 24, 64), ("fp8_gemm_m33n48k96", 33, 48, 96)]:
        A, sa = ref.fp8_quantize_per_tensor(uniform(rng, (M, K)))
        B, sb = ref.fp8_quantize_per_tensor(uniform(rng, (K, N)))
        C0 = uniform(rng, (M, N))
        save(name, A=A, B=B, sa=np.float32(sa), sb=np.float32(sb), C=ref.gemm_fp8_e4m3(A, B, sa, sb), C0=C0,
             C_ab=ref.gemm_fp8_e4m3(A, B, sa, sb, C0, alpha=0.5, beta=2.0))


def scheduler_trace():
    """Step-by-step record of the reference's own Scheduler (src/runtime/scheduler.cpp) on a mixed workload
    in the style of tests/test_scheduler.cpp (MixedWorkloadHitsHighOccupancy, AdmissionStallsOnOOM): more
    requests than the active set holds, a pool small enough to stall admission, random EOS flags."""
    import json
    if not ref_available():
        raise SystemExit("oracle/_ref/liblh_ref.so missing: run `make -C oracle ref` first")
    lib = Checker("lhr").lib
    lib.lhr_cm_create.restype = C.c_void_p
    lib.lhr_sched_create.restype = C.c_void_p
    lib.lhr_sched_last_step_occupancy.restype = C.c_double
    num_blocks, block_size, max_concurrent, n_requests = 24, 4, 6, 40
    L = Layout(num_blocks, block_size, 2, 8)
    m = C.c_void_p(lib.lhr_cm_create(C.byref(L)))
    sch = C.c_void_p(lib.lhr_sched_create(m, max_concurrent))
    rng = np.random.default_rng(4242)
    reqs = [(int(rng.integers(1, 14)), int(rng.integers(1, 9))) for _ in range(n_requests)]
    ids = [lib.lhr_sched_submit(sch, p, n) for p, n in reqs]
    steps = []
    while lib.lhr_sched_has_work(sch):
        n = lib.lhr_sched_prepare_step(sch)
        if n == 0:
            break
        mb = lib.lhr_sched_step_max_blocks(sch)
        a_ids, lens, tab = np.zeros(n, np.int32), np.zeros(n, np.int32), np.zeros(n * mb, np.int32)
        lib.lhr_sched_step_view(sch, a_ids.ctypes.data_as(C.c_void_p), lens.ctypes.data_as(C.c_void_p),
                                tab.ctypes.data_as(C.c_void_p))
        flags = (rng.random(n) < 0.08).astype(np.uint8)
        steps.append({"ids": a_ids.tolist(), "seq_lens": lens.tolist(), "max_blocks": int(mb),
                      "tables": tab.reshape(n, mb).tolist(), "queue": lib.lhr_sched_queue_depth(sch),
                      "occupancy": lib.lhr_sched_last_step_occupancy(sch), "free": lib.lhr_cm_num_free(m),
                      "completed": flags.tolist()})
        lib.lhr_sched_commit_step(sch, flags.ctypes.data_as(C.c_void_p), n)
    out = {"num_blocks": num_blocks, "block_size": block_size, "max_concurrent": max_concurrent,
           "requests": reqs, "submitted_ids": ids, "steps": steps,
           "generated": [lib.lhr_sched_generated(sch, i) for i in ids], "free_at_end": lib.lhr_cm_num_free(m)}
    lib.lhr_sched_destroy(sch)
    lib.lhr_cm_destroy(m)
    with open(os.path.join(HERE, "scheduler_trace.json"), "w") as f:
        json.dump(out, f)
    print("wrote scheduler_trace:", len(steps), "steps,", sum(1 for s in steps if s["queue"]), "with a queue")


if __name__ == "__main__":
    if "--fp8" in sys.argv:
        fp8_fixtures()
    elif "--sched" in sys.argv:
        scheduler_trace()
    elif "--asym" in sys.argv:
        asym_fixtures()
    elif "--glue" in sys.argv:        # only the decode-step glue fixtures (the others stay as they are)
        glue_fixtures()
    else:
        main()
        glue_fixtures()
        asym_fixtures()
        fp8_fixtures()
        scheduler_trace()

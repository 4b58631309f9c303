"""GPU parity at the sizes the benchmark workloads are stated at (not scaled-down stand-ins):

* paged int8-KV decode attention: 64 sequences with lengths U[512, 4096] over a 65,536-page pool,
  Hq 32 / Hkv 8 / head_dim 128 / page 16, tables cut from one permutation of the pool;
* W8A8 GEMM 8192 x 8192 x 28672 (per-token int8 activations, per-channel int8 weights): the
  quantisers bit for bit, and the product bit for bit on a contiguous slab of rows plus 64 rows
  sampled across M (the CPU function is exactly linear in M, so rows can be checked one by one);
* one full-width decode layer (d 4096, 32/8 heads of 128, FFN 14336, int4 group 128, batch 32,
  2048 cached tokens per sequence) against the CPU composition of the same operators for three
  of the 32 requests (every operator of the layer works row by row / request by request).

The CPU side is the plain-C restatement of the reference (bit-identical to the compiled reference,
see test_oracle_cpu.py) with its OpenMP harness loops; each case takes seconds of CPU time.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import longhornai_b200 as lb
from cpu_checker import AttnCfg, Checker, Layout, PagedPools
from gpu_util import assert_close, assert_same_bits, dev, host, lb_cfg, lb_layout

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def port():
    c = Checker("lho")
    import os
    c.set_threads(len(os.sched_getaffinity(0)))
    return c


def test_paged_decode_at_the_benchmark_size(port):
    n_req, hq, hkv, d, bs, pool_pages = 64, 32, 8, 128, 16, 65536
    rng = np.random.default_rng(20243)
    lens = rng.integers(512, 4097, size=n_req).astype(np.int32)
    perm = rng.permutation(pool_pages).astype(np.int32)
    max_blocks = 4096 // bs
    tables = np.full((n_req, max_blocks), -1, np.int32)
    used = 0
    for r, l in enumerate(lens):
        nb = (int(l) + bs - 1) // bs
        tables[r, :nb] = perm[used:used + nb]
        used += nb
    L = Layout(pool_pages, bs, hkv, d)
    # K, V ~ N(0, 1), appended on both sides from the same rows
    shp = (pool_pages, hkv, bs, d)
    k = torch.zeros(shp, dtype=torch.int8, device="cuda"); v = torch.zeros_like(k)
    ks = torch.zeros(shp[:3], device="cuda"); vs = torch.zeros_like(ks)
    pools = port.empty_pools_q8(L)
    td = dev(tables)
    kn_all, vn_all, offs, off = [], [], [], 0
    for r, l in enumerate(lens):
        kn = rng.standard_normal((hkv, int(l), d)).astype(np.float32)
        vn = rng.standard_normal((hkv, int(l), d)).astype(np.float32)
        lb.paged_kv_append_q8(k, v, ks, vs, dev(kn), dev(vn), td[r], lb_layout(L), 0, int(l))
        offs.append(off); off += kn.size
        kn_all.append(kn.ravel()); vn_all.append(vn.ravel())
    port.paged_kv_append_q8_batched(pools, np.concatenate(kn_all), np.concatenate(vn_all), np.array(offs, np.int64),
                                    tables, np.zeros(n_req, np.int32), lens, L)
    del kn_all, vn_all
    assert_same_bits(host(ks), pools.ks, "K scales, 64k-page pool")
    assert_same_bits(host(vs), pools.vs, "V scales")
    assert_same_bits(host(k), pools.k, "K pool (1 GiB)")
    assert_same_bits(host(v), pools.v, "V pool (1 GiB)")
    Q = rng.standard_normal((n_req, hq, 1, d)).astype(np.float32)
    cfg = AttnCfg(hq, hkv, 1, d, 1, 0.0, 0, 0)
    c_cfg, c_L = lb_cfg(cfg), lb_layout(L)
    assert lb._cabi.load().lhb_paged_attention_q8_fast_path(C.byref(c_cfg), C.byref(c_L)) == 1
    got = host(lb.paged_attention_q8_batched(dev(Q), k, v, ks, vs, td, dev(lens), lb_cfg(cfg), lb_layout(L)))
    want = port.paged_attention_q8_batched(Q, pools, tables, lens, cfg, L, parallel=True)
    assert_close(got, want, what=f"paged decode, {n_req} sequences, {int(lens.sum())} cached tokens")
    # the entry point that allocates nothing serves the same shape from its fixed arrays
    out = torch.full((n_req, hq, 1, d), float("nan"), device="cuda")
    lb.paged_attention_q8_batched_noalloc(dev(Q), k, v, ks, vs, td, dev(lens), lb_cfg(cfg), lb_layout(L), out)
    assert_close(host(out), want, what="no-alloc entry point at the benchmark size")
    assert lb.default_context().poll() == 0


def test_w8a8_at_the_benchmark_size(port):
    M, K, N = 8192, 8192, 28672
    gen = torch.Generator(device="cuda").manual_seed(20245)
    X = torch.randn(M, K, device="cuda", generator=gen)
    Aq, a_s = lb.q8_quantize_per_row(X)
    rows = np.unique(np.concatenate([np.arange(4000, 4064), np.random.default_rng(5).integers(0, M, 64)]))
    xq, xs = port.q8_quantize_per_row(host(X[torch.from_numpy(rows).cuda()]))
    assert_same_bits(host(Aq)[rows], xq, "per-token int8 activations (sampled rows)")
    assert_same_bits(host(a_s)[rows], xs, "per-token scales")
    del X
    W = torch.randn(K, N, device="cuda", generator=gen) * 0.02
    Bq, b_s = lb.q8_quantize_per_col(W)
    wq, ws = port.q8_quantize_per_col(host(W))
    del W
    Bq_h = host(Bq)
    assert_same_bits(Bq_h, wq, "per-channel int8 weights (235 MB)")
    assert_same_bits(host(b_s), ws, "per-channel scales")
    del wq
    assert lb._cabi.load().lhb_gemm_w8a8_fast_path(M, N, K) == 1
    Cout = lb.gemm_w8a8(Aq, Bq, a_s, b_s)
    torch.cuda.synchronize()
    got = host(Cout[torch.from_numpy(rows).cuda()])
    want = port.par_gemm_w8a8_mslabs(np.ascontiguousarray(host(Aq)[rows]), Bq_h, np.ascontiguousarray(host(a_s)[rows]),
                                     host(b_s), 4)
    assert_same_bits(got, want, f"W8A8 {M}x{K}x{N}: {len(rows)} rows of C")
    assert bool(torch.isfinite(Cout).all())                 # nothing of the 940 MB output is left unwritten
    assert lb.default_context().poll() == 0


def test_full_width_decode_layer_against_cpu_composition(port):
    from longhornai_b200 import decode_step as ds
    from test_gpu_decode_step import cpu_layer

    rng = np.random.default_rng(20244)
    cfg = dict(dim=4096, n_q_heads=32, n_kv_heads=8, head_dim=128, ffn=14336, group=128, theta=500000.0, eps=1e-5)
    n_req, ctx_len, block = 32, 2048, 16
    blocks_per_req = (ctx_len + 1 + block - 1) // block
    num_blocks = n_req * blocks_per_req
    past = np.full(n_req, ctx_len, np.int32)
    L = Layout(num_blocks, block, cfg["n_kv_heads"], cfg["head_dim"])
    acfg = AttnCfg(cfg["n_q_heads"], cfg["n_kv_heads"], 1, cfg["head_dim"], 1, 0.0, 0, 0)
    tables = rng.permutation(num_blocks).astype(np.int32).reshape(n_req, blocks_per_req)
    d, f, G = cfg["dim"], cfg["ffn"], cfg["group"]

    def q4(k, n):
        w = torch.randn(k, n, device="cuda", generator=gen) * (1.0 / np.sqrt(k))
        p, s = lb.q4_quantize_groupwise(w, G)              # bit-exact with the CPU quantiser (tested elsewhere)
        return host(p), host(s)
    gen = torch.Generator(device="cuda").manual_seed(20244)
    w = dict(wq=q4(d, d), wk=q4(d, 1024), wv=q4(d, 1024), wo=q4(d, d), wgu=q4(d, 2 * f), wdown=q4(f, d))
    w["g_attn"] = rng.uniform(0.5, 1.5, d).astype(np.float32)
    w["g_ffn"] = rng.uniform(0.5, 1.5, d).astype(np.float32)
    # a cache that already holds 2048 tokens per request
    pools = port.empty_pools_q8(L)
    kk = rng.standard_normal((n_req, cfg["n_kv_heads"], ctx_len, cfg["head_dim"])).astype(np.float32)
    vv = rng.standard_normal((n_req, cfg["n_kv_heads"], ctx_len, cfg["head_dim"])).astype(np.float32)
    per = kk[0].size
    port.paged_kv_append_q8_batched(pools, kk.ravel(), vv.ravel(), np.arange(n_req, dtype=np.int64) * per, tables,
                                    np.zeros(n_req, np.int32), past, L)
    del kk, vv
    x0 = rng.standard_normal((n_req, d)).astype(np.float32)

    scfg = ds.StepConfig(d, cfg["n_q_heads"], cfg["n_kv_heads"], cfg["head_dim"], f, G, cfg["theta"], False, cfg["eps"])
    layer = ds.LayerWeights.from_quantized(*[(dev(w[k][0]), dev(w[k][1])) for k in ("wq", "wk", "wv", "wo", "wgu", "wdown")],
                                           dev(w["g_attn"]), dev(w["g_ffn"]))
    pools_gpu = ds.KVPools(dev(pools.k), dev(pools.v), dev(pools.ks), dev(pools.vs))
    x = dev(x0.copy())
    buf = ds.StepBuffers.allocate(scfg, n_req, x.device)
    ds.decode_step(x, [layer], [pools_gpu], dev(tables), dev(past), dev(past + 1), scfg, lb_layout(L), lb_cfg(acfg), buf)
    got = host(x)

    sel = np.array([0, 13, 31])
    want = cpu_layer(port, x0[sel].copy(), w, pools, tables[sel], past[sel], cfg, L, acfg)
    # seven chained operators per row, each within the library tolerance of its own inputs
    assert_close(got[sel], want, rtol=3e-3, atol=3e-4, what="full-width decode layer, requests 0, 13, 31")
    err = np.abs(got[sel] - want)
    print(f"full-width layer: max abs err {err.max():.3e}, max |want| {np.abs(want).max():.3f}")
    # the rotated K row and the V row of the new token landed in the cache bit for bit (same inputs
    # up to the projection's tolerance: allow the few int8 codes that sit on a rounding boundary)
    gk, ck = host(pools_gpu.k), pools.k
    for r in sel:
        blk, slot = tables[r, ctx_len // block], ctx_len % block
        diff = np.mean(gk[blk, :, slot] != ck[blk, :, slot])
        assert diff < 5e-3, f"request {r}: {diff:.4f} of the new K bytes differ"
    assert lb.default_context().poll() == 0

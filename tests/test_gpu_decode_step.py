"""GPU: a two-layer decode step (norm, int4 projections, rotary embedding, int8 KV append,
paged attention, SwiGLU MLP, residuals) against the same composition of the CPU checker's
functions, for a ragged batch with permuted block tables."""
import numpy as np
import pytest

from cpu_checker import AttnCfg, Checker, Layout, best_checker
from gpu_util import assert_close, dev, host, lb_cfg, lb_layout

pytestmark = pytest.mark.gpu


def cpu_layer(chk, x, w, pools, tables, past, cfg, L, acfg):
    G = cfg["group"]
    n_req = x.shape[0]
    Hq, Hkv, hd = cfg["n_q_heads"], cfg["n_kv_heads"], cfg["head_dim"]
    h = chk.rmsnorm(x, w["g_attn"], cfg["eps"])
    q = chk.gemm_w4a16_groupwise(h, *w["wq"], G)
    k = chk.gemm_w4a16_groupwise(h, *w["wk"], G)
    v = chk.gemm_w4a16_groupwise(h, *w["wv"], G)
    o = np.empty_like(q)
    for r in range(n_req):
        qr = chk.rope(q[r].reshape(1, Hq, hd), cfg["theta"], 1.0, False, int(past[r]))
        kr = chk.rope(k[r].reshape(1, Hkv, hd), cfg["theta"], 1.0, False, int(past[r]))
        chk.paged_kv_append_q8(pools, kr.reshape(Hkv, 1, hd), v[r].reshape(Hkv, 1, hd), tables[r], L, int(past[r]), 1)
        o[r] = chk.paged_attention_q8(qr.reshape(Hq, 1, hd), pools, tables[r], int(past[r]) + 1, acfg, L).reshape(-1)
    x = chk.gemm_w4a16_groupwise(o, *w["wo"], G, x, alpha=1.0, beta=1.0)
    h = chk.rmsnorm(x, w["g_ffn"], cfg["eps"])
    a = chk.swiglu(chk.gemm_w4a16_groupwise(h, *w["wgu"], G))
    return chk.gemm_w4a16_groupwise(a, *w["wdown"], G, x, alpha=1.0, beta=1.0)


def test_two_layer_decode_step_matches_cpu_composition():
    import torch
    import longhornai_b200 as lb
    from longhornai_b200 import decode_step as ds

    chk = best_checker()
    rng = np.random.default_rng(404)
    cfg = dict(dim=512, n_q_heads=4, n_kv_heads=2, head_dim=128, ffn=768, group=128, theta=500000.0, eps=1e-5)
    n_layers, n_req, block, num_blocks, max_blocks = 2, 3, 16, 24, 4
    past = np.array([5, 16, 37], np.int32)
    L = Layout(num_blocks, block, cfg["n_kv_heads"], cfg["head_dim"])
    acfg = AttnCfg(cfg["n_q_heads"], cfg["n_kv_heads"], 1, cfg["head_dim"], 1, 0.0, 0, 0)
    perm = rng.permutation(num_blocks).astype(np.int32)
    tables = np.full((n_req, max_blocks), -1, np.int32)
    used = 0
    for r in range(n_req):
        nb = (int(past[r]) + 1 + block - 1) // block
        tables[r, :nb] = perm[used:used + nb]
        used += nb

    def wmat(k, n):
        return (rng.standard_normal((k, n)) * (1.0 / np.sqrt(k))).astype(np.float32)

    layers_cpu, pools_cpu = [], []
    for _ in range(n_layers):
        d, f = cfg["dim"], cfg["ffn"]
        raw = dict(wq=wmat(d, d), wk=wmat(d, 256), wv=wmat(d, 256), wo=wmat(d, d), wgu=wmat(d, 2 * f),
                   wdown=wmat(f, d))
        w = {k: chk.q4_quantize_groupwise(v, cfg["group"]) for k, v in raw.items()}
        w["g_attn"] = rng.uniform(0.5, 1.5, d).astype(np.float32)
        w["g_ffn"] = rng.uniform(0.5, 1.5, d).astype(np.float32)
        layers_cpu.append(w)
        # a cache that already holds `past` tokens per request
        pools = chk.empty_pools_q8(L)
        for r in range(n_req):
            kk = rng.standard_normal((cfg["n_kv_heads"], int(past[r]), cfg["head_dim"])).astype(np.float32)
            vv = rng.standard_normal((cfg["n_kv_heads"], int(past[r]), cfg["head_dim"])).astype(np.float32)
            chk.paged_kv_append_q8(pools, kk, vv, tables[r], L, 0, int(past[r]))
        pools_cpu.append(pools)

    x0 = rng.standard_normal((n_req, cfg["dim"])).astype(np.float32)

    # ---- GPU ----
    scfg = ds.StepConfig(cfg["dim"], cfg["n_q_heads"], cfg["n_kv_heads"], cfg["head_dim"], cfg["ffn"], cfg["group"],
                         cfg["theta"], False, cfg["eps"])
    layers_gpu = [ds.LayerWeights.from_quantized(
        *[(dev(w[k][0]), dev(w[k][1])) for k in ("wq", "wk", "wv", "wo", "wgu", "wdown")],
        dev(w["g_attn"]), dev(w["g_ffn"])) for w in layers_cpu]
    pools_gpu = [ds.KVPools(dev(p.k), dev(p.v), dev(p.ks), dev(p.vs)) for p in pools_cpu]
    x = dev(x0.copy())
    buf = ds.StepBuffers.allocate(scfg, n_req, x.device)
    ds.decode_step(x, layers_gpu, pools_gpu, dev(tables), dev(past), dev(past + 1), scfg, lb_layout(L), lb_cfg(acfg), buf)
    got = host(x)

    # ---- CPU composition ----
    want = x0.copy()
    for w, pools in zip(layers_cpu, pools_cpu):
        want = cpu_layer(chk, want, w, pools, tables, past, cfg, L, acfg)

    # the new token's K/V rows landed in the cache bit-exactly in layer 0 (same inputs on both sides)
    assert np.array_equal(host(pools_gpu[0].k), pools_cpu[0].k) or \
        np.mean(host(pools_gpu[0].k) != pools_cpu[0].k) < 1e-3
    # thirteen chained operators: each within 1e-3 of its own inputs, the chain within 5e-3
    assert_close(got, want, rtol=5e-3, atol=5e-4, what="two-layer decode step")
    assert lb.default_context().poll() == 0

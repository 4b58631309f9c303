"""CPU: the decode-step composition (`longhornai_b200.decode_step`) run with the CPU stand-in
for the kernels - single rank against a hand-written composition, and two gloo ranks of the
tensor-parallel step against the single-rank result (bit-identical: column slabs of a GEMM,
heads of attention and replicated norms do not change any sum)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))


def _setup(rng, ds, chk, cfg, n_layers, n_req, past, L, tables):
    """Seeded weights, caches holding `past` tokens, hidden state: the same on every rank."""
    def wmat(k, n):
        return (rng.standard_normal((k, n)) * (1.0 / np.sqrt(k))).astype(np.float32)
    layers, pools = [], []
    for _ in range(n_layers):
        q = lambda w: tuple(torch.from_numpy(a) for a in chk.q4_quantize_groupwise(w, cfg.group))
        d, f = cfg.dim, cfg.ffn
        lw = ds.LayerWeights.from_quantized(q(wmat(d, cfg.q_dim)), q(wmat(d, cfg.kv_dim)), q(wmat(d, cfg.kv_dim)),
                                            q(wmat(cfg.q_dim, d)), q(wmat(d, 2 * f)), q(wmat(f, d)),
                                            torch.from_numpy(rng.uniform(0.5, 1.5, d).astype(np.float32)),
                                            torch.from_numpy(rng.uniform(0.5, 1.5, d).astype(np.float32)))
        layers.append(lw)
        from cpu_checker import Layout
        p = chk.empty_pools_q8(Layout(L.num_blocks, L.block_size, L.n_kv_heads, L.head_dim))
        for r in range(n_req):
            kk = rng.standard_normal((L.n_kv_heads, int(past[r]), L.head_dim)).astype(np.float32)
            vv = rng.standard_normal((L.n_kv_heads, int(past[r]), L.head_dim)).astype(np.float32)
            chk.paged_kv_append_q8(p, kk, vv, tables[r], Layout(L.num_blocks, L.block_size, L.n_kv_heads, L.head_dim),
                                   0, int(past[r]))
        pools.append(ds.KVPools(*(torch.from_numpy(a) for a in (p.k, p.v, p.ks, p.vs))))
    x0 = torch.from_numpy(rng.standard_normal((n_req, cfg.dim)).astype(np.float32))
    return layers, pools, x0


def _problem():
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.dirname(HERE))
    import longhornai_b200  # noqa: F401  (the package imports without a GPU)
    from longhornai_b200 import decode_step as ds
    from longhornai_b200._cabi import PagedAttnCfg, PagedLayout
    from cpu_checker import Checker
    from cpu_ops import CpuOps
    chk = Checker("lho")
    cfg = ds.StepConfig(256, 4, 2, 64, 384, 64, 500000.0, False, 1e-5)
    n_layers, n_req, block, num_blocks, max_blocks = 2, 3, 16, 12, 3
    past = np.array([5, 16, 33], np.int32)
    L = PagedLayout(num_blocks, block, cfg.n_kv_heads, cfg.head_dim)
    acfg = PagedAttnCfg(cfg.n_q_heads, cfg.n_kv_heads, 1, cfg.head_dim, 1, 0.0, 0, 0)
    rng = np.random.default_rng(77)
    perm = rng.permutation(num_blocks).astype(np.int32)
    tables = np.full((n_req, max_blocks), -1, np.int32)
    used = 0
    for r in range(n_req):
        nb = (int(past[r]) + 1 + block - 1) // block
        tables[r, :nb] = perm[used:used + nb]
        used += nb
    layers, pools, x0 = _setup(rng, ds, chk, cfg, n_layers, n_req, past, L, tables)
    return ds, CpuOps(chk), cfg, L, acfg, layers, pools, x0, torch.from_numpy(tables), torch.from_numpy(past)


def _single_rank():
    ds, ops, cfg, L, acfg, layers, pools, x0, tables, past = _problem()
    x = x0.clone()
    buf = ds.StepBuffers.allocate(cfg, x.shape[0], x.device)
    ds.decode_step(x, layers, pools, tables, past, past + 1, cfg, L, acfg, buf, ops=ops)
    return x.numpy(), pools


def test_single_rank_step_equals_hand_composition():
    ds, ops, cfg, L, acfg, layers, pools, x0, tables, past = _problem()
    chk = ops.chk
    got, _ = _single_rank()
    # the same layer written out by hand with the checker's functions, unfused weights
    from cpu_checker import AttnCfg, Layout, PagedPools
    Lc = Layout(L.num_blocks, L.block_size, L.n_kv_heads, L.head_dim)
    ac = AttnCfg(cfg.n_q_heads, cfg.n_kv_heads, 1, cfg.head_dim, 1, 0.0, 0, 0)
    x = x0.numpy().copy()
    for w, kv in zip(layers, pools):
        pp = PagedPools(kv.k.numpy().copy(), kv.v.numpy().copy(), kv.ks.numpy().copy(), kv.vs.numpy().copy())
        h = chk.rmsnorm(x, w.g_attn.numpy(), cfg.eps)
        qkv = chk.gemm_w4a16_groupwise(h, w.wqkv[0].numpy(), w.wqkv[1].numpy(), cfg.group)
        q, k, v = qkv[:, :cfg.q_dim], qkv[:, cfg.q_dim:cfg.q_dim + cfg.kv_dim], qkv[:, cfg.q_dim + cfg.kv_dim:]
        o = np.empty((x.shape[0], cfg.q_dim), np.float32)
        for r in range(x.shape[0]):
            p = int(past[r])
            qr = chk.rope(q[r].reshape(1, cfg.n_q_heads, cfg.head_dim), cfg.rope_theta, 1.0, False, p)
            kr = chk.rope(k[r].reshape(1, cfg.n_kv_heads, cfg.head_dim), cfg.rope_theta, 1.0, False, p)
            chk.paged_kv_append_q8(pp, kr.reshape(cfg.n_kv_heads, 1, cfg.head_dim),
                                   np.ascontiguousarray(v[r]).reshape(cfg.n_kv_heads, 1, cfg.head_dim),
                                   tables[r].numpy(), Lc, p, 1)
            o[r] = chk.paged_attention_q8(qr.reshape(cfg.n_q_heads, 1, cfg.head_dim), pp, tables[r].numpy(), p + 1,
                                          ac, Lc).reshape(-1)
        x = chk.gemm_w4a16_groupwise(o, w.wo[0].numpy(), w.wo[1].numpy(), cfg.group, x, alpha=1.0, beta=1.0)
        h = chk.rmsnorm(x, w.g_ffn.numpy(), cfg.eps)
        a = chk.swiglu(chk.gemm_w4a16_groupwise(h, w.wgu[0].numpy(), w.wgu[1].numpy(), cfg.group))
        x = chk.gemm_w4a16_groupwise(a, w.wdown[0].numpy(), w.wdown[1].numpy(), cfg.group, x, alpha=1.0, beta=1.0)
    assert np.array_equal(got, x)


def _tp_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ds, ops, cfg, L, acfg, layers, pools, x0, tables, past = _problem()
    from longhornai_b200 import sharding as sh
    from longhornai_b200._cabi import PagedAttnCfg, PagedLayout
    want, want_pools = _single_rank()
    lc = ds.local_config(cfg, world)
    layers_r = [ds.shard_layer(w, cfg, rank, world) for w in layers]
    pools_r = [ds.KVPools(*sh.shard_kv_pools(p.k, p.v, p.ks, p.vs, rank, world)) for p in pools]
    Lr = PagedLayout(L.num_blocks, L.block_size, lc.n_kv_heads, lc.head_dim)
    acr = PagedAttnCfg(lc.n_q_heads, lc.n_kv_heads, 1, lc.head_dim, 1, 0.0, 0, 0)
    x = x0.clone()
    buf = ds.TPBuffers.allocate(cfg, world, x.shape[0], x.device)
    ds.decode_step_tp(x, layers_r, pools_r, tables, past, past + 1, cfg, Lr, acr, buf, rank, world, dist, ops=ops)
    lo, hi = sh.kv_head_range(cfg.n_kv_heads, rank, world)
    ok_x = np.array_equal(x.numpy(), want)
    ok_kv = all(np.array_equal(pr.k.numpy(), pw.k.numpy()[:, lo:hi]) and
                np.array_equal(pr.vs.numpy(), pw.vs.numpy()[:, lo:hi]) for pr, pw in zip(pools_r, want_pools))
    ret[rank] = (ok_x, ok_kv)
    dist.barrier()
    dist.destroy_process_group()


def test_tensor_parallel_step_world2_equals_single_rank():
    world, port = 2, 29600 + os.getpid() % 300
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_tp_worker, args=(world, port, ret), nprocs=world, join=True)
        assert all(ret[r] == (True, True) for r in range(world)), dict(ret)

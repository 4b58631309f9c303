"""One rank of the multi-GPU check of the peer-memory exchange; launched by
test_gpu_peer_exchange.py with torch.distributed.run, one process per GPU.

(a) the exchange alone: random slabs, many calls back to back over alternating matrices, each
    rank's copy must equal the concatenation of all ranks' slabs;
(b) the sharded decode step with the push all-gather against the same step with library
    all-gathers and against the single-rank step: residual stream and KV pools bit-identical,
    eager and replayed from a CUDA graph;
(c) the N-sharded W8A8 GEMM whose epilogue stores its tiles into every rank's matrix: each rank's
    copy bit-identical to the unsharded product computed locally.
Prints PEER_EXCHANGE_OK on rank 0 when every rank passed."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import longhornai_b200 as lb  # noqa: E402
from longhornai_b200 import decode_step as ds, peer, sharding as sh  # noqa: E402


def slab(rows, w, call, rank):
    g = torch.Generator(device="cuda").manual_seed(1000 * call + rank)
    return torch.randn(rows, w, device="cuda", generator=g)


def exchange_alone(rank, world):
    shapes = {"a": (32, 4096), "b": (32, 2 * 14336 // 2), "c": (3, 64 * world)}
    pg = peer.PeerGather(shapes, rank, world, dist)
    order = ["a", "b", "c", "b", "a", "c"]
    for call in range(48):
        name = order[call % len(order)]
        rows, cols = shapes[name]
        w = cols // world
        out = pg.gather(slab(rows, w, call, rank), name)
        if call % 5 == 0 or call > 40:          # most calls run back to back without a host sync
            want = torch.cat([slab(rows, w, call, p) for p in range(world)], dim=1)
            assert torch.equal(out, want), f"rank {rank}: call {call} ({name}) differs"
            dist.barrier()                      # nobody overwrites a matrix a slower rank still compares
    pg.check()
    pg.close(dist)


def sharded_step(rank, world, n_req=5):
    """n_req = 5: the projections run on the GEMV kernel and the exchanges are separate launches;
    n_req = 40: they run on the tensor-core kernel, whose epilogue pushes the residual slabs itself."""
    cfg = ds.StepConfig(1024, 8, 4, 128, 2048, 128, 500000.0, False, 1e-5)
    n_layers, bs, bpr = 2, 16, 8
    nb = n_req * bpr
    L = lb.PagedLayout(nb, bs, cfg.n_kv_heads, cfg.head_dim)
    acfg = lb.PagedAttnCfg(cfg.n_q_heads, cfg.n_kv_heads, 1, cfg.head_dim, 1, 0.0, 0, 0)
    g = torch.Generator(device="cuda").manual_seed(3)
    tables = torch.from_numpy(np.random.default_rng(0).permutation(nb).astype(np.int32).reshape(n_req, bpr)).cuda()
    past = torch.tensor([5, 16, 37, 100, 64] * (n_req // 5), dtype=torch.int32, device="cuda")
    cur = past + 1

    def rnd(k, n):
        return torch.randn(k, n, device="cuda", generator=g) * (1.0 / np.sqrt(k))
    layers, pools = [], []
    for _ in range(n_layers):
        layers.append(ds.LayerWeights.quantize(
            cfg, rnd(1024, 1024), rnd(1024, 512), rnd(1024, 512), rnd(1024, 1024), rnd(1024, 4096), rnd(2048, 1024),
            torch.rand(1024, device="cuda", generator=g) + 0.5, torch.rand(1024, device="cuda", generator=g) + 0.5))
        shape = (nb, cfg.n_kv_heads, bs, cfg.head_dim)
        pools.append(ds.KVPools(
            torch.randint(-127, 128, shape, dtype=torch.int8, device="cuda", generator=g),
            torch.randint(-127, 128, shape, dtype=torch.int8, device="cuda", generator=g),
            torch.rand(shape[:3], device="cuda", generator=g) * 0.02 + 0.005,
            torch.rand(shape[:3], device="cuda", generator=g) * 0.02 + 0.005))
    x0 = torch.randn(n_req, 1024, device="cuda", generator=g)

    def clone(ps):
        return [ds.KVPools(p.k.clone(), p.v.clone(), p.ks.clone(), p.vs.clone()) for p in ps]
    # single rank
    pools1 = clone(pools)
    x1 = x0.clone()
    ds.decode_step(x1, layers, pools1, tables, past, cur, cfg, L, acfg, ds.StepBuffers.allocate(cfg, n_req, x1.device))
    # sharded, library all-gathers
    lc = ds.local_config(cfg, world)
    lw = [ds.shard_layer(w, cfg, rank, world) for w in layers]
    shard = lambda: [ds.KVPools(*[t.contiguous() for t in sh.shard_kv_pools(p.k, p.v, p.ks, p.vs, rank, world)])
                     for p in pools]
    Lr = lb.PagedLayout(nb, bs, lc.n_kv_heads, lc.head_dim)
    ar = lb.PagedAttnCfg(lc.n_q_heads, lc.n_kv_heads, 1, lc.head_dim, 1, 0.0, 0, 0)
    pools2 = shard()
    x2 = x0.clone()
    ds.decode_step_tp(x2, lw, pools2, tables, past, cur, cfg, Lr, ar, ds.TPBuffers.allocate(cfg, world, n_req, x2.device),
                      rank, world, dist)
    # sharded, push all-gather over peer memory
    pg = peer.PeerGather(ds.TPBuffers.peer_shapes(cfg, n_req), rank, world, dist)
    buf = ds.TPBuffers.allocate(cfg, world, n_req, x0.device, peer=pg)
    buf.fused_push = n_req >= 17        # the fused form needs the tensor-core kernel
    pools3 = shard()
    buf.x.copy_(x0)
    ds.decode_step_tp(buf.x, lw, pools3, tables, past, cur, cfg, Lr, ar, buf, rank, world, dist)
    torch.cuda.synchronize()
    # the GEMV kernel's result does not depend on how N is sharded; the tensor-core kernel deals its K
    # ranges out by the shard's tile count, so its sharded sums may differ from the unsharded ones in the
    # last place - the two sharded forms run the same GEMMs and must agree exactly either way
    assert torch.equal(buf.x, x2), f"rank {rank}: peer-gather step differs from the library-gather step"
    if n_req < 17:
        assert torch.equal(x2, x1), f"rank {rank}: sharded step differs from the single-rank step"
    else:
        err = (x2 - x1).abs().max().item()
        assert err <= 1e-4 + 1e-3 * x1.abs().max().item(), f"rank {rank}: sharded step off by {err}"
    lo, hi = sh.kv_head_range(cfg.n_kv_heads, rank, world)
    for a, b, c in zip(pools3, pools2, pools1):
        assert torch.equal(a.k, b.k) and torch.equal(a.v, b.v) and torch.equal(a.ks, b.ks) and torch.equal(a.vs, b.vs)
        if n_req < 17:
            assert torch.equal(a.k, c.k[:, lo:hi]) and torch.equal(a.vs, c.vs[:, lo:hi])
    # the same step as a CUDA graph, replayed
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            buf.x.copy_(x0)
            ds.decode_step_tp(buf.x, lw, pools3, tables, past, cur, cfg, Lr, ar, buf, rank, world, dist)
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(5):
        graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(buf.x, x2), f"rank {rank}: graph replay of the peer-gather step differs"
    pg.check()
    assert lb.default_context().poll() == 0
    del graph
    pg.close(dist)


def w8a8_sharded(rank, world):
    M, K, n_local = 640, 1024, 512                  # M ends inside a tile
    N = n_local * world
    g = torch.Generator(device="cuda").manual_seed(77)      # every rank draws the same operands
    Aq, a_s = lb.q8_quantize_per_row(torch.randn(M, K, device="cuda", generator=g))
    Bq, b_s = lb.q8_quantize_per_col(torch.randn(K, N, device="cuda", generator=g) * 0.02)
    want = lb.gemm_w8a8(Aq, Bq, a_s, b_s, alpha=0.75)
    pg = peer.PeerGather({"c": (M, N), "d": (M, N)}, rank, world, dist)
    if rank == 0:
        print(f"PEER_MAPPING {pg.mapping}", flush=True)
    lo = rank * n_local
    Bl, bl = Bq[:, lo:lo + n_local].contiguous(), b_s[lo:lo + n_local].contiguous()
    for call in range(6):
        name = "cd"[call % 2]
        pg.tensor(name).fill_(-3.0)
        torch.cuda.synchronize()
        dist.barrier()                              # nobody's fill lands on top of a peer's tiles
        out = pg.gemm_w8a8_sharded(Aq, Bl, a_s, bl, name, alpha=0.75)
        torch.cuda.synchronize()
        dist.barrier()                              # every rank's stores are complete
        assert torch.equal(out, want), f"rank {rank}: sharded W8A8 call {call} differs from the unsharded product"
    assert lb.default_context().poll() == 0
    pg.close(dist)


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    exchange_alone(rank, world)
    sharded_step(rank, world)
    sharded_step(rank, world, n_req=40)
    w8a8_sharded(rank, world)
    ok = torch.ones(1, device="cuda")
    dist.all_reduce(ok)
    if rank == 0 and int(ok.item()) == world:
        print("PEER_EXCHANGE_OK", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

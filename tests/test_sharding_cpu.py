"""World-size-2 gloo test of the multi-GPU host logic: N-sharded GEMMs and
KV-head-sharded attention reassemble to the unsharded result.  The per-rank
compute is done by the CPU checker here (test infrastructure standing in for the
kernels, which need a GPU); what is under test is the sharding, the gathered
layout and the collective."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))


def _worker(rank, world, port, ret):
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.dirname(HERE))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from cpu_checker import AttnCfg, Checker, Layout, PagedPools
    from longhornai_b200 import sharding as sh
    chk = Checker("lho")
    rng = np.random.default_rng(5)                       # same data on every rank
    K, N, G, M = 256, 128, 64, 3
    W = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    A = rng.standard_normal((M, K)).astype(np.float32)
    p, s = chk.q4_quantize_groupwise(W, G)
    full = chk.gemm_w4a16_groupwise(A, p, s, G)
    pl, sl = sh.shard_w4(torch.from_numpy(p), torch.from_numpy(s), rank, world)
    local = torch.from_numpy(chk.gemm_w4a16_groupwise(A, pl.numpy(), sl.numpy(), G))
    got = sh.assemble_columns(sh.all_gather_columns(local, world, dist)).numpy()
    ok_w4 = np.array_equal(got, full)                    # column slabs are bit-identical
    q, qs = chk.q8_quantize_per_col(W)
    full8 = chk.gemm_w8a16_perchannel(A, q, qs)
    ql, qsl = sh.shard_w8(torch.from_numpy(q), torch.from_numpy(qs), rank, world)
    local8 = torch.from_numpy(chk.gemm_w8a16_perchannel(A, ql.numpy(), qsl.numpy()))
    ok_w8 = np.array_equal(sh.assemble_columns(sh.all_gather_columns(local8, world, dist)).numpy(), full8)

    # attention by KV head
    qh, kvh, d, bs, nblk = 8, 4, 16, 4, 12
    L, cfg = Layout(nblk, bs, kvh, d), AttnCfg(qh, kvh, 1, d, 1, 0.0, 0, 0)
    lens = [13, 6]
    tables = np.array([[3, 1, 7, 0], [5, 2, -1, -1]], np.int32)
    pools = chk.empty_pools_q8(L)
    for r, l in enumerate(lens):
        kn = rng.standard_normal((kvh, l, d)).astype(np.float32)
        vn = rng.standard_normal((kvh, l, d)).astype(np.float32)
        chk.paged_kv_append_q8(pools, kn, vn, tables[r], L, 0, l)
    Q = rng.standard_normal((2, qh, 1, d)).astype(np.float32)
    seq_lens = np.array(lens, np.int32)
    O_full = chk.paged_attention_q8_batched(Q, pools, tables, seq_lens, cfg, L)
    k, v, ks, vs = sh.shard_kv_pools(*(torch.from_numpy(x) for x in (pools.k, pools.v, pools.ks, pools.vs)),
                                     rank, world)
    Ql = sh.shard_q_heads(torch.from_numpy(Q), kvh, rank, world)
    Ll, cfgl = Layout(nblk, bs, kvh // world, d), AttnCfg(qh // world, kvh // world, 1, d, 1, 0.0, 0, 0)
    O_loc = chk.paged_attention_q8_batched(Ql.numpy(), PagedPools(k.numpy(), v.numpy(), ks.numpy(), vs.numpy()),
                                           tables, seq_lens, cfgl, Ll)
    O = sh.assemble_heads(sh.all_gather_columns(torch.from_numpy(O_loc), world, dist)).numpy()
    ok_attn = np.array_equal(O, O_full)
    ret[rank] = (ok_w4, ok_w8, ok_attn)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharding_reassembles_to_the_unsharded_result():
    world = 2
    port = 29500 + os.getpid() % 2000
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        assert dict(ret) == {0: (True, True, True), 1: (True, True, True)}


def test_shard_ranges_and_alignment():
    from longhornai_b200 import sharding as sh
    assert sh.column_range(14336, 3, 8) == (5376, 7168)
    assert sh.kv_head_range(8, 1, 4) == (2, 4)
    import pytest
    with pytest.raises(ValueError):
        sh.column_range(100, 0, 8)
    with pytest.raises(ValueError):
        sh.kv_head_range(8, 0, 3)


def _fd_worker(rank, world, port, ret):
    sys.path.insert(0, os.path.dirname(HERE))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import socket
    import tempfile
    from longhornai_b200.peer import pass_descriptors
    # every rank owns a file with its own content; the peers must end up reading that content through
    # the descriptor they were sent (a descriptor number means nothing in another process)
    f = tempfile.TemporaryFile()
    f.write(f"owned by rank {rank}".encode())
    f.flush()
    sock = socket.socket(socket.AF_UNIX, socket.SOCK_DGRAM)
    addr = f"\0lhb-test-{os.getpid()}-{rank}"
    sock.bind(addr)
    sock.settimeout(30.0)
    addrs = [None] * world
    dist.all_gather_object(addrs, addr)
    got = pass_descriptors(sock, f.fileno(), rank, addrs)
    ok = sorted(got) == [p for p in range(world) if p != rank]
    for p, fd in got.items():
        ok = ok and os.pread(fd, 64, 0) == f"owned by rank {p}".encode()
        os.close(fd)
    sock.close()
    ret[rank] = ok
    dist.barrier()
    dist.destroy_process_group()


def test_descriptors_reach_every_other_rank():
    """The exchange that shares driver-managed GPU allocations between the ranks' processes, with
    ordinary files standing in for the allocations: three ranks, one datagram per pair and direction."""
    world = 3
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_fd_worker, args=(world, 31500 + os.getpid() % 2000, ret), nprocs=world, join=True)
        assert all(ret[r] for r in range(world)), dict(ret)

"""The decode-attention entry point that allocates no device memory.

Some hosts of this library cannot let it call cudaMalloc (all of HBM already
belongs to their own pools, or their rules forbid allocation after start-up), so
they have no context to pass.  lhb_paged_attention_q8_batched_noalloc serves
them from fixed scratch arrays inside the library image.  This test calls it
through the C ABI twice in a row (the second call finds the first call's
leftovers in the shared arrays) and compares each result with the
context-based entry point and with the CPU checker on the same inputs, within
the library tolerance;
it also checks that sizes beyond the fixed arrays are refused with a message.

Collected last on purpose, so a run that stops at the first failure has already
run every other test; it passes alone in a fresh process as well.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import longhornai_b200 as lb
from cpu_checker import AttnCfg, Layout, PagedPools, best_checker
from gpu_util import assert_close, host

pytestmark = pytest.mark.gpu


def make_case(seed, lens, hq=32, hkv=8, d=128, bs=16, nblk=700):
    g = torch.Generator(device="cuda").manual_seed(seed)
    rng = np.random.default_rng(seed)
    L = lb.PagedLayout(nblk, bs, hkv, d)
    cfg = lb.PagedAttnCfg(hq, hkv, 1, d, 1, 0.0, 0, 0)
    n = len(lens)
    max_blocks = max((l + bs - 1) // bs for l in lens)
    perm = rng.permutation(nblk).astype(np.int32)
    tables = np.full((n, max_blocks), -1, np.int32)
    used = 0
    for r, l in enumerate(lens):
        nb = (l + bs - 1) // bs
        tables[r, :nb] = perm[used:used + nb]
        used += nb
    shp = (nblk, hkv, bs, d)
    k = torch.zeros(shp, dtype=torch.int8, device="cuda"); v = torch.zeros_like(k)
    ks = torch.zeros(shp[:3], device="cuda"); vs = torch.zeros_like(ks)
    td = torch.from_numpy(tables).cuda()
    for r, l in enumerate(lens):
        kn = torch.randn(hkv, l, d, device="cuda", generator=g)
        vn = torch.randn(hkv, l, d, device="cuda", generator=g)
        lb.paged_kv_append_q8(k, v, ks, vs, kn, vn, td[r], L, 0, l)
    Q = torch.randn(n, hq, 1, d, device="cuda", generator=g)
    sl = torch.tensor(lens, dtype=torch.int32, device="cuda")
    return Q, k, v, ks, vs, td, sl, cfg, L


def test_noalloc_entry_point_matches_context_entry_point_twice():
    lib = lb._cabi.load()
    assert hasattr(lib, "lhb_paged_attention_q8_batched_noalloc")
    for seed, lens in ((1, [1500, 33, 700, 16, 2049]), (2, [260, 4000, 5])):
        Q, k, v, ks, vs, td, sl, cfg, L = make_case(seed, lens)
        want = lb.paged_attention_q8_batched(Q, k, v, ks, vs, td, sl, cfg, L)
        # and the CPU restatement of the reference on the same pools, so that a fault shared by both
        # entry points (they run the same kernel) cannot pass unnoticed
        chk = best_checker()
        Lc, cc = Layout(L.num_blocks, L.block_size, L.n_kv_heads, L.head_dim), AttnCfg(cfg.n_q_heads, cfg.n_kv_heads, 1,
                                                                                       cfg.head_dim, 1, 0.0, 0, 0)
        want_cpu = chk.paged_attention_q8_batched(host(Q), PagedPools(host(k), host(v), host(ks), host(vs)), host(td),
                                                  host(sl), cc, Lc)
        for call in (1, 2):                              # two calls in a row share the fixed arrays
            got = torch.full_like(Q, float("nan"))      # caller-owned output, poisoned
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]
            lb.paged_attention_q8_batched_noalloc(Q, k, v, ks, vs, td, sl, cfg, L, got)
            torch.cuda.synchronize()
            assert torch.cuda.mem_get_info()[0] >= free_before, "the call took device memory"
            assert torch.isfinite(got).all()
            assert_close(host(got), host(want), what=f"no-alloc entry point, case {seed}, call {call}")
            assert_close(host(got), want_cpu, what=f"no-alloc entry point against the CPU checker, case {seed}, call {call}")


def test_noalloc_entry_point_rejects_sizes_beyond_its_fixed_arrays():
    lib = lb._cabi.load()
    Q, k, v, ks, vs, td, sl, cfg, L = make_case(3, [40, 20])
    n_req = 600                                           # 600 * 8 KV heads > 4096 counters
    big_Q = torch.zeros(n_req, 32, 1, 128, device="cuda")
    big_O = torch.zeros_like(big_Q)
    big_t = td[:1].repeat(n_req, 1).contiguous()
    big_sl = sl[:1].repeat(n_req).contiguous()
    with pytest.raises(lb.LhbError) as e:
        lb.paged_attention_q8_batched_noalloc(big_Q, k, v, ks, vs, big_t, big_sl, cfg, L, big_O)
    assert e.value.status == lb._cabi.ERR_SCRATCH
    assert b"4096" in lib.lhb_last_error()
    # a shape outside the decode fast path is refused, not served by a fallback
    cfg2 = lb.PagedAttnCfg(32, 8, 2, 128, 1, 0.0, 0, 0)
    with pytest.raises(lb.LhbError) as e:
        lb.paged_attention_q8_batched_noalloc(torch.zeros(2, 32, 2, 128, device="cuda"), k, v, ks, vs, td, sl,
                                              cfg2, L, torch.zeros(2, 32, 2, 128, device="cuda"))
    assert e.value.status == lb._cabi.ERR_UNSUPPORTED

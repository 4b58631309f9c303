"""CPU suite for the boundary: the C-ABI library loads without a GPU, exports
every symbol the header declares, validates arguments before touching CUDA, and
the cache manager's host bookkeeping reproduces the reference's allocation
order (golden trace from the reference's own CacheManager)."""
import ctypes as C
import os
import re

import pytest

import golden_io as gio
from longhornai_b200 import _cabi, build as lb_build
from longhornai_b200 import DeviceCacheManager, PagedLayout

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    lb_build.build()
    return _cabi.load()


def header_symbols():
    text = open(os.path.join(ROOT, "include", "lhb200.h")).read()
    return sorted(set(re.findall(r"\b(lhb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(lib):
    names = header_symbols()
    assert len(names) >= 40
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/lhb200.h but not exported"
    # and the Python binding table covers the header one to one
    assert set(_cabi.SIGNATURES) == set(names)


def test_no_torch_dependency_in_the_library():
    import subprocess
    out = subprocess.run(["ldd", _cabi.LIB_PATH], capture_output=True, text=True).stdout
    assert "torch" not in out and "libcuda.so" not in out and "c10" not in out


def test_argument_validation_comes_before_cuda(lib):
    fake = C.c_void_p(16)      # non-null, never dereferenced: validation fails first
    assert lib.lhb_gemm_w4a16_groupwise(None, fake, fake, fake, fake, 1, 16, 16, 16, 1.0, 0.0, None) == _cabi.ERR_NULL
    assert lib.lhb_gemm_w4a16_groupwise(fake, fake, fake, fake, fake, 1, 16, 15, 5, 1.0, 0.0, None) == _cabi.ERR_BAD_SHAPE
    assert lib.lhb_gemm_w4a16_groupwise(fake, fake, fake, fake, fake, 1, 16, 32, 12, 1.0, 0.0, None) == _cabi.ERR_BAD_SHAPE
    assert lib.lhb_gemm_w8a8(fake, fake, fake, fake, fake, fake, 4, 0, 8, 1.0, 0.0, None) == _cabi.ERR_BAD_SHAPE
    assert lib.lhb_q4_quantize_groupwise(fake, fake, fake, fake, 7, 4, 7, None) == _cabi.ERR_BAD_SHAPE
    L = PagedLayout(4, 4, 2, 8)
    cfg = _cabi.PagedAttnCfg(3, 2, 1, 8, 1, 0.0, 0, 0)      # 3 % 2 != 0
    assert lib.lhb_paged_attention_q8_batched(fake, fake, fake, fake, fake, fake, fake, 4, fake, 1, fake,
                                              C.byref(cfg), C.byref(L), None) == _cabi.ERR_BAD_SHAPE
    assert lib.lhb_status_string(_cabi.ERR_TIMEOUT) == b"device-side wait timed out"
    # the entry points added around the decode step, fp8 and asymmetric int4
    assert lib.lhb_rmsnorm(fake, fake, fake, fake, 2, 0, 1e-5, None) == _cabi.ERR_BAD_SHAPE
    assert lib.lhb_rmsnorm(None, fake, fake, fake, 2, 8, 1e-5, None) == _cabi.ERR_NULL
    assert lib.lhb_rope(fake, fake, 2, 2, 7, 1e4, 1.0, 1, 0, None) == _cabi.ERR_BAD_SHAPE        # odd head_dim
    assert lib.lhb_rope_decode_batched(fake, fake, None, 2, 2, 8, 1e4, 1.0, 1, None) == _cabi.ERR_NULL
    assert lib.lhb_swiglu(fake, fake, fake, 2, 0, None) == _cabi.ERR_BAD_SHAPE
    assert lib.lhb_gemm_w4a16_groupwise_prologue(fake, fake, 3, fake, 1e-5, fake, fake, fake, 4, 16, 128, 128, 1.0, 0.0,
                                                 None) == _cabi.ERR_BAD_SHAPE                     # unknown prologue
    assert lib.lhb_gemm_w4a16_groupwise_prologue(fake, fake, 1, None, 1e-5, fake, fake, fake, 4, 16, 128, 128, 1.0, 0.0,
                                                 None) == _cabi.ERR_NULL                          # rmsnorm needs gamma
    assert lib.lhb_gemm_w4a16_groupwise_prologue(fake, fake, 2, None, 0.0, fake, fake, fake, 1, 16, 128, 128, 1.0, 0.0,
                                                 None) == _cabi.ERR_UNSUPPORTED                   # one row: separate calls
    assert lib.lhb_qkv_rope_append_q8_decode(fake, fake, 10, fake, fake, fake, fake, fake, fake, 4, fake, 1, 2, C.byref(L),
                                             1e4, 1.0, 0, None) == _cabi.ERR_BAD_SHAPE            # row stride too small
    assert lib.lhb_fp8_dequantize(fake, fake, fake, fake, 2, 8, 3, None) == _cabi.ERR_BAD_SHAPE   # mode out of range
    assert lib.lhb_gemm_fp8_e4m3(fake, fake, fake, 1.0, 1.0, fake, 4, 0, 8, 1.0, 0.0, None) == _cabi.ERR_BAD_SHAPE
    assert lib.lhb_q4a_quantize_groupwise(fake, fake, fake, fake, fake, 7, 4, 7, None) == _cabi.ERR_BAD_SHAPE
    assert lib.lhb_gemm_w4a16_asym(fake, fake, fake, fake, fake, fake, 1, 16, 32, 12, 1.0, 0.0, None) == _cabi.ERR_BAD_SHAPE
    assert lib.lhb_gemm_w4a16_asym_fast_path(1, 14336, 4096, 128) == 1 and lib.lhb_gemm_w4a16_asym_fast_path(1, 256, 256, 64) == 0
    assert lib.lhb_gemm_fp8_fast_path(256, 256, 256) == 1 and lib.lhb_gemm_fp8_fast_path(8, 256, 256) == 0
    assert lib.lhb_gemm_w4a16_groupwise_peer(fake, fake, fake, fake, fake, 32, 256, 128, 128, 1.0, 0.0, fake, fake, fake,
                                             2, 2, 100, None) == _cabi.ERR_BAD_SHAPE              # rank out of range
    assert lib.lhb_gemm_w4a16_groupwise_peer(fake, fake, fake, fake, fake, 4, 256, 128, 128, 1.0, 0.0, fake, fake, fake,
                                             0, 2, 100, None) == _cabi.ERR_UNSUPPORTED            # too few rows
    assert lib.lhb_gemm_w4a16_fast_path(512, 14336, 4096, 128) == 1 and lib.lhb_gemm_w4a16_fast_path(2000, 14336, 4096, 128) == 0


def test_fast_path_predicates(lib):
    assert lib.lhb_gemm_w4a16_fast_path(1, 14336, 4096, 128) == 1
    assert lib.lhb_gemm_w4a16_fast_path(32, 14336, 4096, 128) == 1
    assert lib.lhb_gemm_w4a16_fast_path(1, 20, 24, 4) == 0        # generic kernel shapes
    assert lib.lhb_gemm_w8a16_fast_path(16, 4096, 4096) == 1
    assert lib.lhb_gemm_w8a16_fast_path(16, 4095, 4096) == 0


def test_cache_manager_bookkeeping_matches_reference_trace():
    trace = gio.cache_manager_trace()
    cm = DeviceCacheManager(PagedLayout(8, 4, 2, 16), max_requests=4, max_blocks_per_req=16, detached=True)
    r0 = cm.create_request()
    ok = cm.ensure_capacity(r0, 9)
    assert ["r0", r0, int(ok), cm.block_table(r0), cm.num_free_blocks()] == trace[0]
    r1 = cm.create_request()
    ok = cm.ensure_capacity(r1, 13)
    assert ["r1", r1, int(ok), cm.block_table(r1), cm.num_free_blocks()] == trace[1]
    ok = cm.ensure_capacity(r1, 40)                    # out of blocks: nothing changes
    assert ["r1_oom", r1, int(ok), cm.block_table(r1), cm.num_free_blocks()] == trace[2]
    cm.release_request(r0)
    r2 = cm.create_request()                           # id recycled, blocks reused LIFO
    ok = cm.ensure_capacity(r2, 16)
    assert ["r2", r2, int(ok), cm.block_table(r2), cm.num_free_blocks()] == trace[3]
    shared = cm.block_table(r1)[0]
    ok = cm.reference_block(r2, 5, shared)
    assert ["r2_ref", r2, int(ok), cm.block_table(r2), cm.refcount(shared)] == trace[4]


def test_cache_manager_refcounts_and_release():
    # tests/test_cache_manager.cpp:25-94 of the reference, re-expressed
    cm = DeviceCacheManager(PagedLayout(4, 4, 1, 8), max_requests=4, max_blocks_per_req=8, detached=True)
    assert cm.num_free_blocks() == 4 and cm.num_total_blocks() == 4
    r1, r2 = cm.create_request(), cm.create_request()
    assert cm.ensure_capacity(r1, 4)
    shared = cm.block_table(r1)[0]
    assert cm.refcount(shared) == 1
    assert cm.reference_block(r2, 0, shared)
    assert cm.refcount(shared) == 2
    cm.release_request(r1)
    assert cm.refcount(shared) == 1 and cm.num_free_blocks() == 3
    cm.release_request(r2)
    assert cm.refcount(shared) == 0 and cm.num_free_blocks() == 4
    b = cm.allocate_block()
    cm.retain_block(b)
    cm.release_block(b)
    assert cm.refcount(b) == 1
    cm.release_block(b)
    cm.release_block(b)                                # double release is ignored
    assert cm.num_free_blocks() == 4


def _replay_scheduler(trace, manager, sched, check_step):
    ids = [sched.submit(p, n) for p, n in trace["requests"]]
    assert ids == trace["submitted_ids"]
    for want in trace["steps"]:
        assert sched.has_work()
        step = sched.prepare_step()
        assert step.ids == want["ids"]
        assert sched.queue_depth() == want["queue"]
        assert abs(sched.last_step_occupancy() - want["occupancy"]) < 1e-12
        assert manager.num_free_blocks() == want["free"]
        for rid, ln, row in zip(step.ids, want["seq_lens"], want["tables"]):
            assert manager.seq_len(rid) == ln
            assert manager.block_table(rid) == [b for b in row if b >= 0]
        check_step(step, want)
        sched.commit_step(want["completed"])
    assert not sched.has_work() or sched.prepare_step().n_active() == 0
    assert [sched.generated(i) for i in ids] == trace["generated"]
    assert manager.num_free_blocks() == trace["free_at_end"]


def test_scheduler_follows_the_reference_step_by_step():
    """The scheduler over a detached (host-only) cache manager reproduces a recorded run of the reference's
    own Scheduler: admissions, stalls on a full pool, retirements, per-step ids / lengths / block tables."""
    import json
    import longhornai_b200 as lb
    trace = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "scheduler_trace.json")))
    L = lb.PagedLayout(trace["num_blocks"], trace["block_size"], 2, 8)
    mgr = lb.DeviceCacheManager(L, max_requests=64, max_blocks_per_req=8, detached=True)
    sched = lb.DeviceScheduler(mgr, trace["max_concurrent"])
    _replay_scheduler(trace, mgr, sched, lambda step, want: None)
    sched.close()
    mgr.close()

"""The push all-gather of the tensor-parallel step (csrc/peer_gather.cu).

On one GPU: the single-rank form through peer.PeerGather; the two-rank data layout and the
bounded wait through the C-ABI with both "ranks'" buffers on the same device - rank 0 is launched
alone, its wait for rank 1 runs out after 50 ms and is reported, then rank 1's launch finds rank
0's arrival already counted and completes.  With two or more GPUs: two processes, real peer
mappings, the exchange alone and the whole sharded layer against the library all-gather form
(bit-identical)."""
import ctypes as C
import os
import subprocess
import sys

import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from longhornai_b200 import _cabi  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("rows,cols", [(1, 16), (32, 4096), (32, 14336), (5, 1000), (256, 8192)])
def test_single_rank_gather_is_a_copy(rows, cols):
    from longhornai_b200 import peer
    pg = peer.PeerGather({"a": (rows, cols), "b": (rows, cols)}, 0, 1, None)
    gen = torch.Generator(device="cuda").manual_seed(rows * 131 + cols)
    for i in range(4):
        src = torch.randn(rows, cols, device="cuda", generator=gen)
        name = "ab"[i & 1]
        out = pg.gather(src, name)
        assert torch.equal(out, src)
    pg.check()
    assert int(pg._state[0].item()) != 0 and int(pg._state[1].item()) == 0
    pg.close()


def test_shareable_allocation_maps_twice_and_unmaps():
    """lhb_peer_alloc_shareable / lhb_peer_open_fd / lhb_peer_unmap inside one process: the descriptor
    maps the same memory a second time, stores through one mapping are read through the other."""
    lib = _cabi.load()
    from longhornai_b200.peer import _DeviceView
    base, fd, mapped = C.c_void_p(), C.c_int(-1), C.c_size_t(0)
    n = 3 * 1024 * 1024 + 512
    assert lib.lhb_peer_alloc_shareable(C.byref(base), n, C.byref(fd), C.byref(mapped)) == _cabi.OK, lib.lhb_last_error()
    assert mapped.value >= n and fd.value >= 0 and base.value % (2 << 20) == 0
    second = C.c_void_p()
    assert lib.lhb_peer_open_fd(fd.value, mapped.value, C.byref(second)) == _cabi.OK, lib.lhb_last_error()
    os.close(fd.value)
    assert second.value not in (None, base.value)
    a = torch.as_tensor(_DeviceView(base.value, n), device="cuda")
    b = torch.as_tensor(_DeviceView(second.value, n), device="cuda")
    assert int(a.count_nonzero().item()) == 0                  # zero-filled
    pattern = torch.arange(n, device="cuda", dtype=torch.int64).mul_(2654435761).bitwise_and_(255).to(torch.uint8)
    a.copy_(pattern)
    torch.cuda.synchronize()
    assert torch.equal(b, pattern)
    del a, b
    torch.cuda.synchronize()
    assert lib.lhb_peer_unmap(second, mapped.value) == _cabi.OK
    assert lib.lhb_peer_unmap(base, mapped.value) == _cabi.OK
    assert lib.lhb_peer_open_fd(-1, mapped.value, C.byref(second)) != _cabi.OK
    assert lib.lhb_peer_alloc_shareable(C.byref(base), 0, C.byref(fd), C.byref(mapped)) != _cabi.OK


def _tables(bufs, flags):
    dev = bufs[0].device
    return (torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device=dev),
            torch.tensor([f.data_ptr() for f in flags], dtype=torch.int64, device=dev))


@pytest.mark.parametrize("rows,w", [(3, 8), (32, 2048), (32, 7168)])
def test_two_rank_layout_and_bounded_wait_on_one_device(rows, w):
    lib = _cabi.load()
    gen = torch.Generator(device="cuda").manual_seed(7 * rows + w)
    full = [torch.zeros(rows, 2 * w, device="cuda") for _ in range(2)]
    flags = [torch.zeros(2, dtype=torch.int32, device="cuda") for _ in range(2)]
    state = [torch.zeros(4, dtype=torch.int32, device="cuda") for _ in range(2)]
    slab = [torch.randn(rows, w, device="cuda", generator=gen) for _ in range(2)]
    dst, flg = _tables(full, flags)
    stream = torch.cuda.current_stream().cuda_stream

    def launch(rank, timeout_ms):
        return lib.lhb_peer_allgather_cols(slab[rank].data_ptr(), rows, w, dst.data_ptr(), flg.data_ptr(),
                                           state[rank].data_ptr(), rank, 2, timeout_ms, stream)
    # rank 0 alone: its slab lands in both copies, nothing arrives from rank 1 -> reported, not hung
    assert launch(0, 50) == _cabi.OK
    assert lib.lhb_peer_status(state[0].data_ptr(), stream) == _cabi.ERR_TIMEOUT
    assert b"rank 1" in lib.lhb_last_error()
    assert int(state[0][2].item()) == 2
    for f in full:
        assert torch.equal(f[:, :w], slab[0]) and not f[:, w:].any()
    # rank 1 next: rank 0's arrival is already counted, so its wait ends at once
    assert launch(1, 1000) == _cabi.OK
    assert lib.lhb_peer_status(state[1].data_ptr(), stream) == _cabi.OK
    want = torch.cat(slab, dim=1)
    for f in full:
        assert torch.equal(f, want)
    cpp = int(state[0][0].item())
    assert cpp >= 1 and flags[0].tolist() == [cpp, cpp] and flags[1].tolist() == [cpp, cpp]
    assert int(state[1][0].item()) == cpp and int(state[0][1].item()) == 0


def test_argument_validation():
    lib = _cabi.load()
    fake = C.c_void_p(256)
    assert lib.lhb_peer_allgather_cols(fake, 4, 6, fake, fake, fake, 0, 2, 100, None) == _cabi.ERR_BAD_SHAPE   # width % 4
    assert lib.lhb_peer_allgather_cols(fake, 4, 8, fake, fake, fake, 2, 2, 100, None) == _cabi.ERR_BAD_SHAPE   # rank
    assert lib.lhb_peer_allgather_cols(fake, 4, 8, fake, fake, fake, 0, 2, 0, None) == _cabi.ERR_BAD_SHAPE     # no limit
    assert lib.lhb_peer_allgather_cols(None, 4, 8, fake, fake, fake, 0, 2, 100, None) == _cabi.ERR_NULL
    assert lib.lhb_peer_allgather_cols(C.c_void_p(260), 4, 8, fake, fake, fake, 0, 2, 100, None) == _cabi.ERR_MISALIGNED


@pytest.mark.timeout(600)
@pytest.mark.parametrize("mapping", ["vmm", "cudaIpc"])
def test_two_processes_two_gpus(mapping):
    """Both ways of sharing the buffers: driver-managed allocations passed as file descriptors (the
    default) and cudaIpc handles (LHB_PEER_VMM=0, also what a failed descriptor exchange falls back to)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0", LHB_PEER_VMM="1" if mapping == "vmm" else "0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29731" if mapping == "vmm" else "29732", os.path.join(ROOT, "tests", "peer_exchange_worker.py")]
    res = subprocess.run(cmd, env=env, cwd=ROOT, capture_output=True, text=True, timeout=540)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "PEER_EXCHANGE_OK" in res.stdout
    assert f"PEER_MAPPING {mapping}" in res.stdout, res.stdout[-2000:]

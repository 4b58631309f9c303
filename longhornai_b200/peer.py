"""Peer-memory buffers and the push all-gather of the tensor-parallel decode step
(csrc/peer_gather.cu).  One process per GPU on one machine; `torch.distributed` is used once, at
set-up, to pass the buffers' 64-byte handles around - the exchange itself is one kernel launch per
rank that stores into the peers' memory over NVLink and waits (bounded) for their stores.

The reference has no multi-device path (src/runtime/scheduler.hpp:47 drives one model on one
device); this file serves only this library's sharded step.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _cabi


class _DeviceView:
    """Lets torch wrap device memory it did not allocate (CUDA array interface, version 2)."""

    def __init__(self, ptr: int, n_bytes: int):
        self.__cuda_array_interface__ = {"shape": (n_bytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class PeerGather:
    """A set of named fp32 matrices [rows, cols] that exist once per rank at the same place in a
    peer-visible allocation, plus the arrival counters of the exchange.  `gather(local, name)` fills
    matrix `name` on every rank from the ranks' column slabs.

    `shapes`: {name: (rows, cols)}; every rank passes the same dict.  `dist` is torch.distributed
    with an initialised default group whose ranks share the machine (unused when world == 1)."""

    def __init__(self, shapes: dict, rank: int, world: int, dist, device=None, timeout_ms: int = 2000):
        self.lib = _cabi.load()
        self.rank, self.world, self.timeout_ms = rank, world, timeout_ms
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self._offsets, off = {}, 256                       # counters live in the first 256 bytes
        assert world <= 64
        for name, (rows, cols) in shapes.items():
            assert cols % (4 * world) == 0, "column slabs must be whole 16-byte pieces"
            self._offsets[name] = (off, rows, cols)
            off += (rows * cols * 4 + 255) // 256 * 256
        self.n_bytes = off
        base = C.c_void_p()
        _cabi.check(self.lib.lhb_peer_alloc(C.byref(base), off), "lhb_peer_alloc")
        self.base = base.value
        handle = (C.c_ubyte * 64)()
        _cabi.check(self.lib.lhb_peer_export(self.base, handle), "lhb_peer_export")
        handles = [bytes(handle)] * world
        if world > 1:
            dist.all_gather_object(handles, bytes(handle))
        self._mapped = []
        bases = []
        try:
            for p in range(world):
                if p == rank:
                    bases.append(self.base)
                    continue
                ptr = C.c_void_p()
                raw = (C.c_ubyte * 64).from_buffer_copy(handles[p])
                _cabi.check(self.lib.lhb_peer_open(raw, C.byref(ptr)), "lhb_peer_open")
                self._mapped.append(ptr.value)
                bases.append(ptr.value)
        except Exception:
            for ptr in self._mapped:                       # leave nothing mapped or allocated behind
                self.lib.lhb_peer_close(ptr)
            self.lib.lhb_peer_free(self.base)
            self.base = None
            raise
        self._bases = list(bases)                          # host copy: rank -> base of that rank's allocation here
        self._keep = _DeviceView(self.base, off)
        self._bytes = torch.as_tensor(self._keep, device=self.device)
        self._flag_table = torch.tensor(bases, dtype=torch.int64, device=self.device)
        self._dst_tables = {name: torch.tensor([b + o for b in bases], dtype=torch.int64, device=self.device)
                            for name, (o, _, _) in self._offsets.items()}
        self._state = torch.zeros(4, dtype=torch.int32, device=self.device)
        self._last = None
        torch.cuda.synchronize(self.device)
        if world > 1:
            dist.barrier()                                 # every rank has mapped every buffer

    def tensor(self, name: str) -> torch.Tensor:
        """This rank's copy of matrix `name` (a view of the peer-visible allocation)."""
        o, rows, cols = self._offsets[name]
        return self._bytes[o:o + rows * cols * 4].view(torch.float32).view(rows, cols)

    def gather(self, local: torch.Tensor, name: str) -> torch.Tensor:
        """`local` [rows, cols/world] is this rank's column slab of matrix `name`; on return of the
        launch (stream order) this rank's copy of the matrix holds every rank's slab."""
        o, rows, cols = self._offsets[name]
        w = cols // self.world
        assert local.is_cuda and local.dtype == torch.float32 and local.is_contiguous()
        assert tuple(local.shape) == (rows, w), (tuple(local.shape), (rows, w))
        assert name != self._last or self.world == 1, "consecutive gathers must fill different matrices"
        self._last = name
        stream = torch.cuda.current_stream(self.device).cuda_stream
        _cabi.check(self.lib.lhb_peer_allgather_cols(local.data_ptr(), rows, w, self._dst_tables[name].data_ptr(),
                                                     self._flag_table.data_ptr(), self._state.data_ptr(), self.rank,
                                                     self.world, self.timeout_ms, stream), "lhb_peer_allgather_cols")
        return self.tensor(name)

    def gemm_w4a16_gather(self, A, packed, scales, group: int, C: torch.Tensor, name: str, alpha=1.0, beta=0.0, ctx=None):
        """C [rows, cols/world] = alpha * A @ dequant(packed, scales) + beta * C on this rank's column shard of
        the weight, and matrix `name` on every rank receives all ranks' results: the GEMM's own epilogue
        stores over NVLink where the tensor-core kernel serves the shape, otherwise GEMM and gather()."""
        from . import kernels as K
        o, rows, cols = self._offsets[name]
        w = cols // self.world
        assert tuple(C.shape) == (rows, w) and C.is_contiguous() and C.dtype == torch.float32
        assert name != self._last or self.world == 1, "consecutive gathers must fill different matrices"
        h = (ctx or K.default_context()).handle
        stream = torch.cuda.current_stream(self.device).cuda_stream
        rc = self.lib.lhb_gemm_w4a16_groupwise_peer(h, A.data_ptr(), packed.data_ptr(), scales.data_ptr(), C.data_ptr(),
                                                    rows, w, A.shape[1], group, float(alpha), float(beta),
                                                    self._dst_tables[name].data_ptr(), self._flag_table.data_ptr(),
                                                    self._state.data_ptr(), self.rank, self.world, self.timeout_ms, stream)
        if rc == _cabi.ERR_UNSUPPORTED:
            K.gemm_w4a16_groupwise(A, packed, scales, group, C=C, alpha=alpha, beta=beta, ctx=ctx)
            return self.gather(C, name)
        _cabi.check(rc, "lhb_gemm_w4a16_groupwise_peer")
        self._last = name
        return self.tensor(name)

    def gemm_w8a8_sharded(self, Aq, Bq, a_scales, b_scales, name: str, alpha: float = 1.0, ctx=None) -> torch.Tensor:
        """N-sharded gemm_w8a8 (lhb_gemm_w8a8_sharded): this rank's weight slab Bq [K, cols/world] against the
        replicated activations Aq [rows, K]; the tensor-core kernel's epilogue stores each finished tile into
        columns [rank * w, (rank + 1) * w) of matrix `name` on every rank while its main loop runs on.  Returns
        this rank's copy of the matrix; it is complete once every rank's stream has passed its own call (follow
        it with a stream-ordered collective, or synchronise and barrier)."""
        from . import kernels as K
        o, rows, cols = self._offsets[name]
        w = cols // self.world
        assert tuple(Aq.shape)[0] == rows and tuple(Bq.shape) == (Aq.shape[1], w), (tuple(Aq.shape), tuple(Bq.shape))
        full = (C.c_void_p * self.world)(*[b + o for b in self._bases])
        h = (ctx or K.default_context()).handle
        stream = torch.cuda.current_stream(self.device).cuda_stream
        _cabi.check(self.lib.lhb_gemm_w8a8_sharded(h, Aq.data_ptr(), Bq.data_ptr(), a_scales.data_ptr(),
                                                   b_scales.data_ptr(), full, self.rank, self.world, rows, w,
                                                   Aq.shape[1], float(alpha), stream), "lhb_gemm_w8a8_sharded")
        self._last = name
        return self.tensor(name)

    def check(self) -> None:
        """Synchronises the current stream and raises if a wait of any gather so far gave up."""
        stream = torch.cuda.current_stream(self.device).cuda_stream
        _cabi.check(self.lib.lhb_peer_status(self._state.data_ptr(), stream), "lhb_peer_status")

    def close(self, dist=None) -> None:
        """Unmaps the peers' buffers and frees this rank's (after a barrier, when `dist` is given, so
        that no peer still writes into it)."""
        if self.base is None:
            return
        torch.cuda.synchronize(self.device)
        if dist is not None:
            dist.barrier()
        for ptr in self._mapped:
            self.lib.lhb_peer_close(ptr)
        self._mapped = []
        if dist is not None:
            dist.barrier()
        self._bytes = None
        self.lib.lhb_peer_free(self.base)
        self.base = None

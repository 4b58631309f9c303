"""Peer-memory buffers and the push all-gather of the tensor-parallel decode step
(csrc/peer_gather.cu, csrc/peer_vmm.cu).  One process per GPU on one machine; `torch.distributed` is
used once, at set-up, to agree on how the buffers are shared - file descriptors of driver-managed
allocations sent over Unix sockets (mapped with large pages everywhere, which kernels that stream
into several peers need), else 64-byte cudaIpc handles - the exchange itself is one kernel launch
per rank that stores into the peers' memory over NVLink and waits (bounded) for their stores.

The reference has no multi-device path (src/runtime/scheduler.hpp:47 drives one model on one
device); this file serves only this library's sharded step.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _cabi


def _use_vmm() -> bool:
    """LHB_PEER_VMM=0 keeps every buffer on the 64-byte-handle mappings."""
    import os
    return os.environ.get("LHB_PEER_VMM", "1") != "0"


def pass_descriptors(sock, fd: int, rank: int, addresses: list) -> dict:
    """Sends file descriptor `fd` to every other rank's datagram socket (`addresses[p]`, this rank's
    own being the bound `sock`) and receives theirs: {rank: descriptor}.  One SCM_RIGHTS datagram per
    pair and direction, the sender's rank as payload; nothing blocks on a peer being ready because
    datagrams queue at the receiver."""
    import array
    import socket
    import struct

    for p, addr in enumerate(addresses):
        if p != rank:
            sock.sendmsg([struct.pack("i", rank)], [(socket.SOL_SOCKET, socket.SCM_RIGHTS, array.array("i", [fd]))], 0, addr)
    got = {}
    while len(got) < len(addresses) - 1:
        msg, anc, _, _ = sock.recvmsg(16, socket.CMSG_SPACE(array.array("i").itemsize))
        fds = array.array("i")
        for level, kind, data in anc:
            if level == socket.SOL_SOCKET and kind == socket.SCM_RIGHTS:
                fds.frombytes(data[:len(data) - len(data) % fds.itemsize])
        if len(msg) != 4 or len(fds) != 1:
            raise OSError("a descriptor datagram arrived without its descriptor")
        got[struct.unpack("i", msg)[0]] = fds[0]
    return got


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
        self._mapped = []                                  # (address, mapped bytes or None) of the peers' buffers here
        self.base, self._own_bytes = None, None
        self.mapping_note = ""                             # why the large-page mappings were not used, if they were not
        bases = self._map_shareable(dist) if world > 1 and _use_vmm() else None
        self.mapping = "vmm" if bases is not None else "cudaIpc"
        if bases is None:
            bases = self._map_handles(dist)
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

    def _map_handles(self, dist) -> list:
        """This rank's buffer from cudaMalloc, the peers' through their 64-byte handles."""
        rank, world = self.rank, self.world
        base = C.c_void_p()
        _cabi.check(self.lib.lhb_peer_alloc(C.byref(base), self.n_bytes), "lhb_peer_alloc")
        self.base, self._own_bytes = base.value, None
        handle = (C.c_ubyte * 64)()
        _cabi.check(self.lib.lhb_peer_export(self.base, handle), "lhb_peer_export")
        handles = [bytes(handle)] * world
        if world > 1:
            dist.all_gather_object(handles, bytes(handle))
        bases = []
        try:
            for p in range(world):
                if p == rank:
                    bases.append(self.base)
                    continue
                ptr = C.c_void_p()
                raw = (C.c_ubyte * 64).from_buffer_copy(handles[p])
                _cabi.check(self.lib.lhb_peer_open(raw, C.byref(ptr)), "lhb_peer_open")
                self._mapped.append((ptr.value, None))
                bases.append(ptr.value)
        except Exception:
            self._release()                                # leave nothing mapped or allocated behind
            raise
        return bases

    def _map_shareable(self, dist):
        """This rank's buffer from the virtual-memory-management calls, mapped with large pages in every
        process: the file descriptors travel over Unix datagram sockets in the abstract namespace (one
        datagram from every rank to every other).  Returns None - with nothing left mapped, on every rank
        alike - when some rank could not do it; the caller then uses the 64-byte handles."""
        import os
        import socket

        rank, world = self.rank, self.world
        base, fd, mapped = C.c_void_p(), C.c_int(-1), C.c_size_t(0)
        rc = self.lib.lhb_peer_alloc_shareable(C.byref(base), self.n_bytes, C.byref(fd), C.byref(mapped))
        sock, addr = None, None
        why = "" if rc == _cabi.OK else f"rank {rank}: lhb_peer_alloc_shareable: {_cabi.last_error()}"
        if rc == _cabi.OK:
            try:
                sock = socket.socket(socket.AF_UNIX, socket.SOCK_DGRAM)
                addr = f"\0lhb-peer-{os.getpid()}-{rank}-{id(self):x}"
                sock.bind(addr)
                sock.settimeout(60.0)
            except OSError as e:
                rc, why = _cabi.ERR_UNSUPPORTED, f"rank {rank}: Unix socket: {e}"
        mine = (rc, addr, int(mapped.value), why)
        everyone = [mine] * world
        dist.all_gather_object(everyone, mine)
        got, ok = {}, all(e[0] == _cabi.OK for e in everyone)
        if ok:
            self.base, self._own_bytes = base.value, int(mapped.value)
            try:
                got = pass_descriptors(sock, fd.value, rank, [e[1] for e in everyone])
            except OSError as e:
                ok, why = False, f"rank {rank}: passing descriptors: {e}"
        bases = []
        if ok:
            for p in range(world):
                if p == rank:
                    bases.append(self.base)
                    continue
                ptr = C.c_void_p()
                if self.lib.lhb_peer_open_fd(got[p], everyone[p][2], C.byref(ptr)) != _cabi.OK:
                    ok, why = False, f"rank {rank}: lhb_peer_open_fd: {_cabi.last_error()}"
                    break
                self._mapped.append((ptr.value, everyone[p][2]))
                bases.append(ptr.value)
        for f in list(got.values()) + ([fd.value] if fd.value >= 0 else []):
            os.close(f)                                    # the mappings keep the memory; the descriptors are done
        if sock is not None:
            sock.close()
        flags = [(ok, why)] * world
        dist.all_gather_object(flags, (ok, why))
        if all(f[0] for f in flags):
            return bases
        self.mapping_note = "; ".join(w for _, w in flags if w) or "; ".join(e[3] for e in everyone if e[3])
        if self.base is None and rc == _cabi.OK:
            self.base, self._own_bytes = base.value, int(mapped.value)
        self._release()
        return None

    def _release(self) -> None:
        for ptr, n in self._mapped:
            if n is None:
                self.lib.lhb_peer_close(ptr)
            else:
                self.lib.lhb_peer_unmap(ptr, n)
        self._mapped = []
        if self.base is not None:
            if self._own_bytes is None:
                self.lib.lhb_peer_free(self.base)
            else:
                self.lib.lhb_peer_unmap(self.base, self._own_bytes)
        self.base = None

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
        """Synchronises the current stream and raises if a wait of any gather so far gave up.  After such
        a timeout the ranks' arrival counters no longer agree: close() this object on every rank and
        create a new one before exchanging again."""
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
        mine, self.base = self.base, None
        self._release()                                    # the peers' buffers first
        self.base = mine
        if dist is not None:
            dist.barrier()
        self._bytes = None
        self._release()

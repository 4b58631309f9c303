"""Device-resident cache manager (host mirror of lh::CacheManager over the C ABI).

Method names follow src/runtime/cache_manager.hpp:34-110 of the reference.  The
pools and the batched block tables / seq_lens live in GPU memory and are
exposed as torch tensors that alias the library's allocations (no copies).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _cabi
from ._cabi import PagedLayout, check

K_INVALID_BLOCK = -1


class DeviceCacheManager:
    def __init__(self, layout: PagedLayout, max_requests: int, max_blocks_per_req: int, ctx=None,
                 detached: bool = False):
        """``detached=True`` keeps only the host bookkeeping (no GPU needed)."""
        self.lib = _cabi.load()
        self.layout = layout
        self.max_requests = max_requests
        self.max_blocks_per_req = max_blocks_per_req
        self.ctx = None
        if not detached:
            from .kernels import default_context
            self.ctx = ctx or default_context()
        h = C.c_void_p()
        check(self.lib.lhb_cm_create(self.ctx.handle if self.ctx else None, C.byref(layout),
                                     max_requests, max_blocks_per_req, C.byref(h)), "lhb_cm_create")
        self.handle = h
        self._views = None

    # -- bookkeeping (reference names) --------------------------------------
    def _stream(self):
        if self.ctx is None:
            return None
        import torch
        return C.c_void_p(torch.cuda.current_stream(self.ctx.device).cuda_stream)

    def num_free_blocks(self) -> int:
        return self.lib.lhb_cm_num_free_blocks(self.handle)

    def num_total_blocks(self) -> int:
        return self.lib.lhb_cm_num_total_blocks(self.handle)

    def create_request(self) -> int:
        return self.lib.lhb_cm_create_request(self.handle)

    def release_request(self, rid: int) -> None:
        check(self.lib.lhb_cm_release_request(self.handle, rid, self._stream()), "release_request")

    def ensure_capacity(self, rid: int, seq_len: int) -> bool:
        r = self.lib.lhb_cm_ensure_capacity(self.handle, rid, seq_len, self._stream())
        if r < 0:
            check(r, "ensure_capacity")
        return r == 1

    def set_seq_len(self, rid: int, seq_len: int) -> None:
        check(self.lib.lhb_cm_set_seq_len(self.handle, rid, seq_len, self._stream()), "set_seq_len")

    def reference_block(self, rid: int, logical_idx: int, physical: int) -> bool:
        r = self.lib.lhb_cm_reference_block(self.handle, rid, logical_idx, physical, self._stream())
        if r < 0:
            check(r, "reference_block")
        return r == 1

    def allocate_block(self) -> int:
        return self.lib.lhb_cm_allocate_block(self.handle)

    def release_block(self, physical: int) -> None:
        self.lib.lhb_cm_release_block(self.handle, physical)

    def retain_block(self, physical: int) -> None:
        self.lib.lhb_cm_retain_block(self.handle, physical)

    def refcount(self, physical: int) -> int:
        return self.lib.lhb_cm_refcount(self.handle, physical)

    def seq_len(self, rid: int) -> int:
        return self.lib.lhb_cm_seq_len(self.handle, rid)

    def block_table(self, rid: int) -> list[int]:
        buf = np.empty(self.max_blocks_per_req, np.int32)
        n = self.lib.lhb_cm_block_table(self.handle, rid, buf.ctypes.data_as(C.c_void_p), buf.size)
        return buf[:n].tolist()

    # -- device storage -------------------------------------------------------
    def tensors(self):
        """(k_pool, v_pool, k_scales, v_scales, block_tables, seq_lens) as CUDA tensors
        aliasing the manager's device memory."""
        if self.ctx is None:
            raise RuntimeError("detached cache manager has no device storage")
        if self._views is None:
            import torch
            L = self.layout
            dev = f"cuda:{self.ctx.device}"
            rows = L.num_blocks * L.n_kv_heads * L.block_size

            def view(ptr, nbytes, dtype, shape):
                iface = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}
                holder = type("_DevMem", (), {"__cuda_array_interface__": iface})()
                return torch.as_tensor(holder, device=dev).view(dtype).view(shape)

            shp = (L.num_blocks, L.n_kv_heads, L.block_size, L.head_dim)
            lib, h = self.lib, self.handle
            self._views = (
                view(lib.lhb_cm_k_pool(h), rows * L.head_dim, torch.int8, shp),
                view(lib.lhb_cm_v_pool(h), rows * L.head_dim, torch.int8, shp),
                view(lib.lhb_cm_k_scales(h), rows * 4, torch.float32, shp[:3]),
                view(lib.lhb_cm_v_scales(h), rows * 4, torch.float32, shp[:3]),
                view(lib.lhb_cm_block_tables(h), self.max_requests * self.max_blocks_per_req * 4,
                     torch.int32, (self.max_requests, self.max_blocks_per_req)),
                view(lib.lhb_cm_seq_lens(h), self.max_requests * 4, torch.int32, (self.max_requests,)),
            )
        return self._views

    def close(self):
        if getattr(self, "handle", None):
            self._views = None
            self.lib.lhb_cm_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class ActiveStep:
    """The view `Scheduler::prepare_step` returns (src/runtime/scheduler.hpp:38-45): ids in step order and,
    on a device-backed scheduler, CUDA tensors `block_tables` [n_active, max_blocks_per_req] (padding -1)
    and `seq_lens` [n_active] aliasing the scheduler's device buffers (valid until the next prepare_step)."""

    def __init__(self, ids, block_tables=None, seq_lens=None, max_blocks_per_req=0):
        self.ids = ids
        self.block_tables = block_tables
        self.seq_lens = seq_lens
        self.max_blocks_per_req = max_blocks_per_req

    def n_active(self) -> int:
        return len(self.ids)


class DeviceScheduler:
    """lh::Scheduler (src/runtime/scheduler.hpp:47-105) over a DeviceCacheManager: same admission and
    retirement rules, with the step's dense block tables gathered on the GPU from the manager's resident
    rows instead of rebuilt on the host.  Requests are (prompt length, max_new_tokens)."""

    def __init__(self, manager: DeviceCacheManager, max_concurrent: int):
        self.lib = manager.lib
        self.manager = manager
        self.max_concurrent = max_concurrent
        h = C.c_void_p()
        check(self.lib.lhb_sched_create(manager.handle, max_concurrent, C.byref(h)), "lhb_sched_create")
        self.handle = h
        self._ids = np.zeros(max(1, max_concurrent), np.int32)

    def submit(self, prompt_len: int, max_new_tokens: int) -> int:
        rid = self.lib.lhb_sched_submit(self.handle, int(prompt_len), int(max_new_tokens))
        if rid < 0:
            raise RuntimeError("lhb_sched_submit failed (no free request row)")
        return rid

    def has_work(self) -> bool:
        return bool(self.lib.lhb_sched_has_work(self.handle))

    def queue_depth(self) -> int:
        return self.lib.lhb_sched_queue_depth(self.handle)

    def active_size(self) -> int:
        return self.lib.lhb_sched_active_size(self.handle)

    def last_step_occupancy(self) -> float:
        return float(self.lib.lhb_sched_last_step_occupancy(self.handle))

    def generated(self, rid: int) -> int:
        return self.lib.lhb_sched_generated(self.handle, rid)

    def prepare_step(self) -> ActiveStep:
        n = self.lib.lhb_sched_prepare_step(self.handle, self._ids.ctypes.data_as(C.c_void_p), self._ids.size,
                                            self.manager._stream())
        if n < 0:
            check(n, "lhb_sched_prepare_step")
        ids = self._ids[:n].tolist()
        mb = self.lib.lhb_sched_max_blocks_per_req(self.handle)
        if self.manager.ctx is None or n == 0:
            return ActiveStep(ids, None, None, mb)
        import torch
        dev = f"cuda:{self.manager.ctx.device}"

        def view(ptr, count, shape):
            iface = {"shape": (count * 4,), "typestr": "|u1", "data": (ptr, False), "version": 2}
            holder = type("_DevMem", (), {"__cuda_array_interface__": iface})()
            return torch.as_tensor(holder, device=dev).view(torch.int32).view(shape)
        return ActiveStep(ids, view(self.lib.lhb_sched_block_tables(self.handle), n * mb, (n, mb)),
                          view(self.lib.lhb_sched_seq_lens(self.handle), n, (n,)), mb)

    def commit_step(self, completed) -> None:
        flags = np.ascontiguousarray(np.asarray(completed, dtype=np.uint8))
        check(self.lib.lhb_sched_commit_step(self.handle, flags.ctypes.data_as(C.c_void_p), int(flags.size),
                                             self.manager._stream()), "lhb_sched_commit_step")

    def close(self):
        if getattr(self, "handle", None):
            self.lib.lhb_sched_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

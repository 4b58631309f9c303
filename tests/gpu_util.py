"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

import longhornai_b200 as lb
from cpu_checker import AttnCfg, Layout

# Library tolerance against the reference's fp32-accumulating kernels.
RTOL, ATOL = 1e-3, 1e-4


def dev(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().numpy()


def assert_close(got, want, rtol=RTOL, atol=ATOL, what=""):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    err = np.abs(got - want)
    tol = atol + rtol * np.abs(want)
    bad = ~(err <= tol)
    if bad.any():
        i = np.unravel_index(np.argmax(err - tol), err.shape)
        raise AssertionError(f"{what}: {bad.sum()} / {bad.size} outside |x-y| <= {atol} + {rtol}|y|; "
                             f"worst at {i}: got {got[i]!r} want {want[i]!r} (err {err[i]:.3e})")


def assert_same_bits(got, want, what=""):
    got, want = np.asarray(got), np.asarray(want)
    assert got.shape == want.shape and got.dtype == want.dtype, (what, got.shape, want.shape, got.dtype, want.dtype)
    neq = got.view(np.uint8) != want.view(np.uint8)
    assert not neq.any(), f"{what}: {int(neq.sum())} differing bytes of {neq.size}"


def lb_layout(L: Layout) -> lb.PagedLayout:
    return lb.PagedLayout(L.num_blocks, L.block_size, L.n_kv_heads, L.head_dim)


def lb_cfg(c: AttnCfg) -> lb.PagedAttnCfg:
    return lb.PagedAttnCfg(c.n_q_heads, c.n_kv_heads, c.seq_q, c.head_dim, c.causal, c.scale,
                           c.window, c.chunk)

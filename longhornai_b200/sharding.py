"""Host-side sharding of the path across the GPUs of one box.

GEMM weights shard along N (output columns): packing and quantisation groups
run along K (src/kernels/quant.hpp:52-57 of the reference), so any 16-aligned
column slab of the packed int4 bytes, of the int8 weights and of their scales is
a self-contained weight for the same kernels.  Attention shards by KV head: a
GQA group (`kvh = qh / group`, src/kernels/kvcache_quant.cpp:108-109) stays on
one rank.  Neither sharding needs a data-path exchange; the only collective is
the all-gather that reassembles outputs, in the layout documented below.
"""
from __future__ import annotations

import torch


def column_range(N: int, rank: int, world: int, align: int = 16) -> tuple[int, int]:
    """Columns [lo, hi) owned by `rank`; every shard is a multiple of `align` wide."""
    if N % (world * align):
        raise ValueError(f"N={N} does not split into {world} shards of {align}-aligned width")
    w = N // world
    return rank * w, (rank + 1) * w


def shard_w4(packed: torch.Tensor, scales: torch.Tensor, rank: int, world: int):
    """Compact [K/2, N/g] packed slab and [K/G, N/g] scales of rank `rank`."""
    lo, hi = column_range(packed.shape[1], rank, world)
    return packed[:, lo:hi].contiguous(), scales[:, lo:hi].contiguous()


def shard_w8(Bq: torch.Tensor, scales: torch.Tensor, rank: int, world: int):
    lo, hi = column_range(Bq.shape[1], rank, world)
    return Bq[:, lo:hi].contiguous(), scales[lo:hi].contiguous()


def kv_head_range(n_kv_heads: int, rank: int, world: int) -> tuple[int, int]:
    if n_kv_heads % world:
        raise ValueError(f"{n_kv_heads} KV heads do not split over {world} ranks")
    w = n_kv_heads // world
    return rank * w, (rank + 1) * w


def shard_kv_pools(k, v, ks, vs, rank: int, world: int):
    """Pools [blocks, heads, block, dim] -> this rank's heads, compact."""
    lo, hi = kv_head_range(k.shape[1], rank, world)
    return (k[:, lo:hi].contiguous(), v[:, lo:hi].contiguous(),
            ks[:, lo:hi].contiguous(), vs[:, lo:hi].contiguous())


def shard_q_heads(Q: torch.Tensor, n_kv_heads: int, rank: int, world: int) -> torch.Tensor:
    """Q [n_req, n_q_heads, seq_q, dim] -> the query heads of this rank's KV heads."""
    group = Q.shape[1] // n_kv_heads
    lo, hi = kv_head_range(n_kv_heads, rank, world)
    return Q[:, lo * group:hi * group].contiguous()


def all_gather_columns(local: torch.Tensor, world: int, dist=None) -> torch.Tensor:
    """All-gather per-rank column slabs [..., M, N/g]; returns the gathered buffer
    [g, ..., M, N/g] (rank-major).  `assemble_columns` turns it into [..., M, N]."""
    if world == 1:
        return local.unsqueeze(0)
    out = torch.empty((world,) + tuple(local.shape), dtype=local.dtype, device=local.device)
    if local.is_cuda:
        dist.all_gather_into_tensor(out, local.contiguous())      # NCCL: one fused collective
    else:
        dist.all_gather(list(out.unbind(0)), local.contiguous())  # gloo (CPU tests)
    return out


def assemble_columns(gathered: torch.Tensor) -> torch.Tensor:
    """[g, ..., M, N/g] -> [..., M, N] (a strided copy; only needed where a consumer
    wants the row-major full matrix)."""
    g = gathered.shape[0]
    return torch.cat([gathered[r] for r in range(g)], dim=-1)


def assemble_heads(gathered: torch.Tensor) -> torch.Tensor:
    """Attention outputs [g, n_req, Hq/g, seq_q, d] -> [n_req, Hq, seq_q, d]."""
    g = gathered.shape[0]
    return torch.cat([gathered[r] for r in range(g)], dim=1)

"""One decode step of a Llama-style layer stack on the quantised path.

This is host-side composition only: every arithmetic step is one of the
library's C-ABI calls, in the order the reference's kernels would be called
for a pre-norm decoder layer with grouped-query attention and a SwiGLU MLP:

    h  = rmsnorm(x)                          src/kernels/normalization.hpp:21         } fused into the
    q | k | v = h Wqkv                       gemm_w4a16_groupwise (gemm_quant.hpp:54), one GEMM over
                                             the three projections' columns side by side
    rope(q), rope(k) at each request's position          src/kernels/rope.hpp:19          } one fused
    append k, v to the int8 paged cache      paged_kv_append_q8 (kvcache_quant.hpp:41)    } launch
    o  = paged attention over the cache      paged_attention_q8 (kvcache_quant.hpp:51)
    x += o Wo                                the residual add is beta = 1 of the GEMM
    h  = rmsnorm(x)
    x += swiglu(h Wgu) Wdown                 src/kernels/activation.hpp:34; Wgu = gate || up

`x` is fp32 [n_requests, dim], one new token per request.  All seven
projections are int4 group-wise weights in the reference layout; Wq, Wk, Wv
are stored as one [dim, q_dim + 2 kv_dim] matrix and gate/up as one
[dim, 2 ffn] matrix (any column slab of a packed int4 matrix is itself a valid
weight, so this is only a choice of where the columns live).  Nothing here
allocates inside the step once `StepBuffers` exists, so a step can be captured
into a CUDA graph after one eager run.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import kernels as K
from ._cabi import PagedAttnCfg, PagedLayout


@dataclass
class StepConfig:
    dim: int
    n_q_heads: int
    n_kv_heads: int
    head_dim: int
    ffn: int
    group: int = 128
    rope_theta: float = 500000.0
    rope_interleaved: bool = False      # Llama checkpoints use the half-rotation layout
    eps: float = 1e-5

    @property
    def q_dim(self) -> int:
        return self.n_q_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.n_kv_heads * self.head_dim


@dataclass
class LayerWeights:
    """(packed uint8 [K/2, N], fp32 scales [K/G, N]) per projection, plus the two norm gains."""
    wqkv: tuple         # [dim, q_dim + 2*kv_dim]: q columns, then k, then v
    wo: tuple
    wgu: tuple          # [dim, 2*ffn]: gate columns first, then up ("value") columns
    wdown: tuple
    g_attn: torch.Tensor
    g_ffn: torch.Tensor

    @staticmethod
    def quantize(cfg: StepConfig, wq, wk, wv, wo, wgu, wdown, g_attn, g_ffn) -> "LayerWeights":
        q = lambda w: K.q4_quantize_groupwise(w, cfg.group)
        return LayerWeights(q(torch.cat([wq, wk, wv], dim=1)), q(wo), q(wgu), q(wdown), g_attn, g_ffn)

    @staticmethod
    def from_quantized(wq, wk, wv, wo, wgu, wdown, g_attn, g_ffn) -> "LayerWeights":
        """From already quantised (packed, scales) pairs: q, k, v are joined along the columns."""
        qkv = (torch.cat([wq[0], wk[0], wv[0]], dim=1).contiguous(),
               torch.cat([wq[1], wk[1], wv[1]], dim=1).contiguous())
        return LayerWeights(qkv, wo, wgu, wdown, g_attn, g_ffn)

    def weight_bytes(self) -> int:
        return sum(p.numel() + s.numel() * 4 for p, s in (self.wqkv, self.wo, self.wgu, self.wdown))


@dataclass
class KVPools:
    """int8 pools [num_blocks, n_kv_heads, block_size, head_dim] and fp32 scale pools of one layer."""
    k: torch.Tensor
    v: torch.Tensor
    ks: torch.Tensor
    vs: torch.Tensor

    @staticmethod
    def empty(L: PagedLayout, device) -> "KVPools":
        shape = (L.num_blocks, L.n_kv_heads, L.block_size, L.head_dim)
        return KVPools(torch.zeros(shape, dtype=torch.int8, device=device),
                       torch.zeros(shape, dtype=torch.int8, device=device),
                       torch.zeros(shape[:3], dtype=torch.float32, device=device),
                       torch.zeros(shape[:3], dtype=torch.float32, device=device))


@dataclass
class StepBuffers:
    """Activations of one layer, reused by every layer of the step."""
    h: torch.Tensor
    qkv: torch.Tensor
    q: torch.Tensor
    k: torch.Tensor
    v: torch.Tensor
    o: torch.Tensor
    gu: torch.Tensor
    act: torch.Tensor

    @staticmethod
    def allocate(cfg: StepConfig, n_req: int, device) -> "StepBuffers":
        f = lambda n: torch.empty((n_req, n), dtype=torch.float32, device=device)
        return StepBuffers(f(cfg.dim), f(cfg.q_dim + 2 * cfg.kv_dim), f(cfg.q_dim), f(cfg.kv_dim), f(cfg.kv_dim), f(cfg.q_dim),
                           f(2 * cfg.ffn), f(cfg.ffn))


def decode_layer(x, w: LayerWeights, pools: KVPools, block_tables, past_lens, cur_lens, cfg: StepConfig,
                 L: PagedLayout, acfg: PagedAttnCfg, buf: StepBuffers, ctx=None, ops=K):
    """Updates `x` [n_req, dim] in place.  `past_lens` = tokens already cached per request (the new
    token's position), `cur_lens` = past_lens + 1; both int32 device tensors.  `ops` is the module
    the kernels are taken from (this package's `kernels`; the CPU tests substitute a stand-in to
    exercise the composition without a GPU)."""
    n_req = x.shape[0]
    G = cfg.group
    ops.gemm_w4a16_norm(x, w.g_attn, cfg.eps, *w.wqkv, G, C=buf.qkv, scratch=buf.h, ctx=ctx)
    # one launch: split [q | k | v], rotate q and k at the request's position, q -> buf.q, k and v -> the cache
    ops.qkv_rope_append_q8_decode(buf.qkv, buf.q.view(n_req, cfg.n_q_heads, cfg.head_dim), pools.k, pools.v,
                                  pools.ks, pools.vs, block_tables, past_lens, cfg.n_q_heads, L, cfg.rope_theta,
                                  1.0, cfg.rope_interleaved, ctx=ctx)
    ops.paged_attention_q8_batched(buf.q.view(n_req, cfg.n_q_heads, 1, cfg.head_dim), pools.k, pools.v, pools.ks,
                                 pools.vs, block_tables, cur_lens, acfg, L,
                                 O=buf.o.view(n_req, cfg.n_q_heads, 1, cfg.head_dim), ctx=ctx)
    ops.gemm_w4a16_groupwise(buf.o, *w.wo, G, C=x, alpha=1.0, beta=1.0, ctx=ctx)
    ops.gemm_w4a16_norm(x, w.g_ffn, cfg.eps, *w.wgu, G, C=buf.gu, scratch=buf.h, ctx=ctx)
    ops.gemm_w4a16_swiglu(buf.gu, *w.wdown, G, C=x, alpha=1.0, beta=1.0, scratch=buf.act, ctx=ctx)
    return x


def decode_step(x, layers, pools, block_tables, past_lens, cur_lens, cfg: StepConfig, L: PagedLayout,
                acfg: PagedAttnCfg, buf: StepBuffers, ctx=None, ops=K):
    """All layers in turn; `layers` and `pools` are per-layer lists."""
    for w, kv in zip(layers, pools):
        decode_layer(x, w, kv, block_tables, past_lens, cur_lens, cfg, L, acfg, buf, ctx=ctx, ops=ops)
    return x


def launches_per_layer(n_req: int, tc_min_rows: int = 17) -> int:
    """Kernel launches in one layer (for the bench's launch count): the fused split + rotation +
    append, attention, and 4 GEMMs.  From `tc_min_rows` rows on a GEMM is one digit pass (which also
    applies RMSNorm / SwiGLU) plus one tensor-core launch per slab of 32 rows; below that it is served
    in slabs of 16 rows plus one digit pass when there are more than two rows, and with one or two
    rows the two norms and SwiGLU are launches of their own."""
    if n_req >= tc_min_rows:
        return 2 + 4 * (1 + (n_req + 31) // 32)
    slabs = (n_req + 15) // 16
    last = n_req - (slabs - 1) * 16
    if last <= 2:
        return 5 + 4 * (slabs + (1 if n_req > 2 else 0))
    return 2 + 4 * (slabs + 1)


# ---- tensor-parallel step: projections sharded along N, attention by KV head ----------------

def shard_layer(w: LayerWeights, cfg: StepConfig, rank: int, world: int) -> LayerWeights:
    """This rank's column slabs of every projection.  The fused QKV slab keeps the rank's query
    heads, then its key heads, then its value heads; the gate||up slab keeps the rank's gate
    columns, then its up columns; o and down keep a plain column slab.  Any 16-aligned column
    slab of a packed int4 matrix and its scales is itself a valid weight."""
    from . import sharding as sh
    hd = cfg.head_dim
    ql, qh = sh.kv_head_range(cfg.n_kv_heads, rank, world)
    grp = cfg.n_q_heads // cfg.n_kv_heads

    def cols(pair, ranges):
        p, s = pair
        return (torch.cat([p[:, a:b] for a, b in ranges], dim=1).contiguous(),
                torch.cat([s[:, a:b] for a, b in ranges], dim=1).contiguous())
    q0, k0, v0 = 0, cfg.q_dim, cfg.q_dim + cfg.kv_dim
    wqkv = cols(w.wqkv, [(q0 + ql * grp * hd, q0 + qh * grp * hd), (k0 + ql * hd, k0 + qh * hd),
                         (v0 + ql * hd, v0 + qh * hd)])
    flo, fhi = sh.column_range(cfg.ffn, rank, world)
    wgu = cols(w.wgu, [(flo, fhi), (cfg.ffn + flo, cfg.ffn + fhi)])
    dlo, dhi = sh.column_range(cfg.dim, rank, world)
    return LayerWeights(wqkv, cols(w.wo, [(dlo, dhi)]), wgu, cols(w.wdown, [(dlo, dhi)]), w.g_attn, w.g_ffn)


def local_config(cfg: StepConfig, world: int) -> StepConfig:
    """The per-rank view: 1/world of the heads and of the FFN columns, the full model width."""
    return StepConfig(cfg.dim, cfg.n_q_heads // world, cfg.n_kv_heads // world, cfg.head_dim, cfg.ffn // world,
                      cfg.group, cfg.rope_theta, cfg.rope_interleaved, cfg.eps)


@dataclass
class TPBuffers:
    """Per-rank activations of the sharded step.  `xs` is this rank's column slab of the replicated
    residual stream.  With `peer` (a peer.PeerGather) the full-width matrices live in peer-visible
    memory, `x` is the residual stream the caller must use, and the exchanges are this library's
    push all-gather; without it `g_*` receive library all-gathers in rank-major layout
    [world, n_req, n/world] and a strided copy lays them out."""
    local: StepBuffers
    xs: torch.Tensor
    o_full: torch.Tensor
    act_full: torch.Tensor
    g_o: torch.Tensor
    g_x: torch.Tensor
    g_act: torch.Tensor
    peer: object = None
    x: torch.Tensor = None
    fused_push: bool = False     # with `peer`: the residual GEMMs push their slabs from their own epilogue
                                 # (measured 2 % slower than GEMM + separate push at batch 32: off by default)

    @staticmethod
    def peer_shapes(cfg: StepConfig, n_req: int) -> dict:
        """The matrices a peer.PeerGather must hold for this step."""
        return {"o": (n_req, cfg.q_dim), "x": (n_req, cfg.dim), "act": (n_req, cfg.ffn)}

    @staticmethod
    def allocate(cfg: StepConfig, world: int, n_req: int, device, peer=None) -> "TPBuffers":
        lc = local_config(cfg, world)
        f = lambda *shape: torch.empty(shape, dtype=torch.float32, device=device)
        local = StepBuffers.allocate(lc, n_req, device)
        if peer is not None:
            return TPBuffers(local, f(n_req, cfg.dim // world), peer.tensor("o"), peer.tensor("act"), None, None, None,
                             peer, peer.tensor("x"))
        return TPBuffers(local, f(n_req, cfg.dim // world), f(n_req, cfg.q_dim),
                         f(n_req, cfg.ffn), f(world, n_req, cfg.q_dim // world), f(world, n_req, cfg.dim // world),
                         f(world, n_req, cfg.ffn // world))


def _gather_rows(dst_full, gathered, local, dist):
    """All-gather `local` [n_req, n/world] into `gathered` [world, n_req, n/world], then lay the slabs
    side by side in `dst_full` [n_req, n] (a strided copy: the next GEMM reads row-major activations)."""
    world, n_req, w = gathered.shape
    if world == 1:
        dst_full.copy_(local)
        return
    if local.is_cuda:
        dist.all_gather_into_tensor(gathered, local)
    else:
        dist.all_gather(list(gathered.unbind(0)), local)
    dst_full.view(n_req, world, w).copy_(gathered.transpose(0, 1))


def decode_layer_tp(x, w: LayerWeights, pools: KVPools, block_tables, past_lens, cur_lens, cfg: StepConfig,
                    L: PagedLayout, acfg: PagedAttnCfg, buf: TPBuffers, rank: int, world: int, dist, ctx=None, ops=K,
                    xs_in_sync: bool = False):
    """One layer on rank `rank` of `world`.  `w` is shard_layer(...), `pools`/`L`/`acfg` describe this rank's
    KV heads, `x` [n_req, dim] is replicated and updated in place.  Exchanges: all-gathers of the attention
    output, of the SwiGLU output and (twice) of the residual slabs; nothing else crosses ranks.  After a layer
    `buf.xs` equals this rank's slab of `x`; `xs_in_sync` says that it already does on entry."""
    lc = local_config(cfg, world)
    b = buf.local
    n_req = x.shape[0]
    G = cfg.group
    lo = rank * (cfg.dim // world)
    if buf.peer is not None:
        assert x.data_ptr() == buf.x.data_ptr(), "with peer buffers the residual stream is buf.x"
        gather = lambda dst, g, local, name: buf.peer.gather(local, name)
    else:
        gather = lambda dst, g, local, name: _gather_rows(dst, g, local, dist)
    ops.gemm_w4a16_norm(x, w.g_attn, cfg.eps, *w.wqkv, G, C=b.qkv, scratch=b.h, ctx=ctx)
    ops.qkv_rope_append_q8_decode(b.qkv, b.q.view(n_req, lc.n_q_heads, lc.head_dim), pools.k, pools.v, pools.ks,
                                  pools.vs, block_tables, past_lens, lc.n_q_heads, L, cfg.rope_theta, 1.0,
                                  cfg.rope_interleaved, ctx=ctx)
    ops.paged_attention_q8_batched(b.q.view(n_req, lc.n_q_heads, 1, lc.head_dim), pools.k, pools.v, pools.ks,
                                 pools.vs, block_tables, cur_lens, acfg, L,
                                 O=b.o.view(n_req, lc.n_q_heads, 1, lc.head_dim), ctx=ctx)
    gather(buf.o_full, buf.g_o, b.o, "o")
    if not xs_in_sync:
        buf.xs.copy_(x[:, lo:lo + cfg.dim // world])
    if buf.peer is not None and buf.fused_push:      # the GEMM's epilogue pushes its slab to every rank where it can
        buf.peer.gemm_w4a16_gather(buf.o_full, *w.wo, G, buf.xs, "x", alpha=1.0, beta=1.0, ctx=ctx)
    else:
        ops.gemm_w4a16_groupwise(buf.o_full, *w.wo, G, C=buf.xs, alpha=1.0, beta=1.0, ctx=ctx)
        gather(x, buf.g_x, buf.xs, "x")
    ops.gemm_w4a16_norm(x, w.g_ffn, cfg.eps, *w.wgu, G, C=b.gu, scratch=b.h, ctx=ctx)
    ops.swiglu(b.gu, out=b.act, ctx=ctx)        # its output is what the ranks exchange
    gather(buf.act_full, buf.g_act, b.act, "act")
    if buf.peer is not None and buf.fused_push:
        buf.peer.gemm_w4a16_gather(buf.act_full, *w.wdown, G, buf.xs, "x", alpha=1.0, beta=1.0, ctx=ctx)
    else:
        ops.gemm_w4a16_groupwise(buf.act_full, *w.wdown, G, C=buf.xs, alpha=1.0, beta=1.0, ctx=ctx)
        gather(x, buf.g_x, buf.xs, "x")
    return x


def decode_step_tp(x, layers, pools, block_tables, past_lens, cur_lens, cfg: StepConfig, L: PagedLayout,
                   acfg: PagedAttnCfg, buf: TPBuffers, rank: int, world: int, dist, ctx=None, ops=K):
    for i, (w, kv) in enumerate(zip(layers, pools)):
        decode_layer_tp(x, w, kv, block_tables, past_lens, cur_lens, cfg, L, acfg, buf, rank, world, dist,
                        ctx=ctx, ops=ops, xs_in_sync=i > 0)
    return x

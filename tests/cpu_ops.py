"""A stand-in for `longhornai_b200.kernels` on CPU tensors, backed by the CPU checker.

Test infrastructure only: it lets the CPU suite run the decode-step composition code
(`longhornai_b200.decode_step`, single-rank and tensor-parallel) without a GPU, so that the
host-side logic - buffer views, weight sharding, the layout of the all-gathers - is
exercised with gloo ranks.  Same call signatures as the kernels module, results written in
place into the caller's torch tensors.
"""
import numpy as np
import torch

from cpu_checker import AttnCfg, Checker, Layout, PagedPools


class CpuOps:
    def __init__(self, chk: Checker | None = None):
        self.chk = chk or Checker("lho")

    @staticmethod
    def _np(t):
        return t.numpy() if isinstance(t, torch.Tensor) else np.asarray(t)

    def rmsnorm(self, x, gamma, eps=1e-5, out=None, ctx=None):
        y = self.chk.rmsnorm(self._np(x), self._np(gamma), eps)
        out.copy_(torch.from_numpy(y))
        return out

    def gemm_w4a16_groupwise(self, A, Bp, Bs, G, C=None, alpha=1.0, beta=0.0, ctx=None):
        y = self.chk.gemm_w4a16_groupwise(self._np(A.contiguous()), self._np(Bp), self._np(Bs), G,
                                          self._np(C).copy() if beta != 0.0 else None, alpha=alpha, beta=beta)
        C.copy_(torch.from_numpy(y))
        return C

    def gemm_w4a16_norm(self, x, gamma, eps, Bp, Bs, G, C=None, alpha=1.0, beta=0.0, scratch=None, ctx=None):
        self.rmsnorm(x, gamma, eps, out=scratch)
        return self.gemm_w4a16_groupwise(scratch, Bp, Bs, G, C=C, alpha=alpha, beta=beta)

    def gemm_w4a16_swiglu(self, x, Bp, Bs, G, C=None, alpha=1.0, beta=0.0, scratch=None, ctx=None):
        self.swiglu(x, out=scratch)
        return self.gemm_w4a16_groupwise(scratch, Bp, Bs, G, C=C, alpha=alpha, beta=beta)

    def rope_decode_batched(self, x, positions, theta_base=10000.0, freq_scale=1.0, interleaved=True, ctx=None):
        xn, pos = self._np(x), self._np(positions)
        for r in range(xn.shape[0]):
            xn[r] = self.chk.rope(xn[r:r + 1], theta_base, freq_scale, interleaved, int(pos[r]))[0]
        return x

    def paged_kv_append_q8_batched(self, k_pool, v_pool, k_scales, v_scales, k_new, v_new, block_tables, past_lens,
                                   L, seq_new=1, ctx=None):
        pools = PagedPools(self._np(k_pool), self._np(v_pool), self._np(k_scales), self._np(v_scales))
        Lc = Layout(L.num_blocks, L.block_size, L.n_kv_heads, L.head_dim)
        kn, vn, tb, past = self._np(k_new), self._np(v_new), self._np(block_tables), self._np(past_lens)
        for r in range(kn.shape[0]):
            self.chk.paged_kv_append_q8(pools, kn[r].reshape(L.n_kv_heads, seq_new, L.head_dim),
                                        vn[r].reshape(L.n_kv_heads, seq_new, L.head_dim), tb[r], Lc, int(past[r]),
                                        seq_new)

    def qkv_rope_append_q8_decode(self, qkv, q_out, k_pool, v_pool, k_scales, v_scales, block_tables, positions,
                                  n_q_heads, L, theta_base=10000.0, freq_scale=1.0, interleaved=True, ctx=None):
        """The fused call as the three reference steps it stands for: rope(q), rope(k), append(k, v)."""
        n_req, hd, hkv = qkv.shape[0], L.head_dim, L.n_kv_heads
        qd, kd = n_q_heads * hd, hkv * hd
        q = qkv[:, :qd].contiguous().view(n_req, n_q_heads, hd)
        k = qkv[:, qd:qd + kd].contiguous().view(n_req, hkv, hd)
        v = qkv[:, qd + kd:qd + 2 * kd].contiguous().view(n_req, hkv, hd)
        self.rope_decode_batched(q, positions, theta_base, freq_scale, interleaved)
        self.rope_decode_batched(k, positions, theta_base, freq_scale, interleaved)
        q_out.copy_(q)
        self.paged_kv_append_q8_batched(k_pool, v_pool, k_scales, v_scales, k, v, block_tables, positions, L, 1)
        return q_out

    def paged_attention_q8_batched(self, Q, K_pool, V_pool, K_scales, V_scales, block_tables, seq_lens, cfg, L,
                                   O=None, ctx=None):
        pools = PagedPools(self._np(K_pool), self._np(V_pool), self._np(K_scales), self._np(V_scales))
        Lc = Layout(L.num_blocks, L.block_size, L.n_kv_heads, L.head_dim)
        cc = AttnCfg(cfg.n_q_heads, cfg.n_kv_heads, cfg.seq_q, cfg.head_dim, cfg.causal, cfg.scale, cfg.window,
                     cfg.chunk)
        y = self.chk.paged_attention_q8_batched(self._np(Q.contiguous()), pools, self._np(block_tables),
                                                self._np(seq_lens), cc, Lc)
        O.copy_(torch.from_numpy(y).view_as(O))
        return O

    def swiglu(self, x, out=None, ctx=None):
        out.copy_(torch.from_numpy(self.chk.swiglu(self._np(x))))
        return out

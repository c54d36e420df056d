"""Latent attention: queries and keys/values pass through low-rank latents, and only the kv latent is cached.

Per token the layer computes, from its input h,
    c_q = RMSnorm(W_dq h) * w_q,   q = W_uq c_q  (per head: `dim` unrotated then `rot_dim` rotated numbers)
    [c | k_r] = W_dkv h,           c <- RMSnorm(c) * w_kv,   k_r <- rotate(k_r)   (one row shared by all heads)
and the cache row of the token is [c | k_r].  Keys and values of head h are W_uk[h] c and W_uv[h] c; they are never
built.  With q_abs[h] = W_uk[h]^T q_plain[h] the score is (q_abs[h] . c + rotate(q_r[h]) . k_r) * scale and the head's
output W_uv[h] (sum_j p_j c_j): attention with ONE key/value head whose key rows have kv_rank + rot_dim numbers and
whose value rows are the first kv_rank of them (`BiasedChunkAttention(values_in_keys=True)`: the engine's paged
portion and decode kernels).  The two per-head changes of basis are batched library GEMMs.  The concatenated heads are
multiplied by sigmoid(W_g h) before the output projection.

A layer built with `source` (another LatentAttention) makes no latent of its own: it attends over the source layer's
cache rows - written earlier in the same step - with its own queries, W_uk, W_uv, gate and output projection.

Kernels: csrc/latent_attn.cu (norms + rotation + cache write; query rotation; gate) and csrc/bias_attn.cu.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from compactor_vllm import _native as N
from compactor_vllm.config.constants import RESERVED_BATCH
from compactor_vllm.layers.attention import BiasedChunkAttention
from compactor_vllm.utils.context import get_context


def rotation_frequencies(rot_dim: int, base: float) -> torch.Tensor:
    """inv_freq[i] = base ** (-2 i / rot_dim), i < rot_dim / 2, as 64-bit floats."""
    return torch.tensor([float(base) ** (-2.0 * i / rot_dim) for i in range(rot_dim // 2)], dtype=torch.float64)


def sigmoid_gate(x: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """x * sigmoid(gate), both [T, width] with unit inner stride (row strides free)."""
    T, width = x.shape
    assert gate.shape == x.shape and x.stride(1) == 1 and gate.stride(1) == 1 and gate.dtype == x.dtype
    out = torch.empty((T, width), dtype=x.dtype, device=x.device)
    N.check(N.lib().cvllm_sigmoid_gate(N.ptr(x), x.stride(0), N.ptr(gate), gate.stride(0), N.ptr(out), out.stride(0), T,
                                       width, N.block_dtype_code(x.dtype), N.stream(x.device)), "cvllm_sigmoid_gate")
    return out


class LatentAttention(nn.Module):
    def __init__(self, width: int, heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, q_rank: int,
                 scale: float, rot_base: float, eps: float, source: Optional["LatentAttention"] = None,
                 dtype: Optional[torch.dtype] = None):
        super().__init__()
        self.heads, self.dim, self.rot_dim, self.vdim = int(heads), int(dim), int(rot_dim), int(vdim)
        self.kv_rank, self.q_rank, self.eps = int(kv_rank), int(q_rank), float(eps)
        self.own_latent = source is None
        self.__dict__["source"] = source          # not a submodule: its parameters belong to its own layer
        if source is not None:
            assert (source.kv_rank, source.rot_dim) == (self.kv_rank, self.rot_dim) and source.own_latent
        self.row = self.kv_rank + self.rot_dim     # numbers per cache row
        # the paged attention over the latent rows; a layer without a latent of its own borrows the source's cache views
        self.attn = BiasedChunkAttention(self.heads, 1, self.row, self.kv_rank, scale, values_in_keys=True)
        kv_cols = self.row if self.own_latent else 0
        self.q_off, self.kv_off, self.g_off = 0, (self.q_rank if self.own_latent else -1), self.q_rank + kv_cols
        self.in_proj = nn.Linear(width, self.q_rank + kv_cols + self.heads * self.vdim, bias=False)   # dq | dkv | gate
        self.q_norm = nn.Parameter(torch.ones(self.q_rank, dtype=torch.float32))
        self.kv_norm = nn.Parameter(torch.ones(self.kv_rank, dtype=torch.float32)) if self.own_latent else None
        self.uq_proj = nn.Linear(self.q_rank, self.heads * (self.dim + self.rot_dim), bias=False)
        self.uk = nn.Parameter(torch.empty(self.heads, self.dim, self.kv_rank, dtype=dtype))
        self.uv = nn.Parameter(torch.empty(self.heads, self.vdim, self.kv_rank, dtype=dtype))
        self.o_proj = nn.Linear(self.heads * self.vdim, width, bias=False)
        self.register_buffer("inv_freq", rotation_frequencies(self.rot_dim, rot_base), persistent=False)

    def _cache(self) -> BiasedChunkAttention:
        a = self.attn
        if not self.own_latent and a.k_cache is None:
            s = self.source.attn
            a.k_cache, a.page_table, a.bh_seq_lens, a.page_size = s.k_cache, s.page_table, s.bh_seq_lens, s.page_size
        assert a.k_cache is not None, "KV cache must be initialized"
        return a

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        ctx = get_context()
        attn = self._cache()
        T = h.shape[0]
        H, D, R, Dv, r = self.heads, self.dim, self.rot_dim, self.vdim, self.kv_rank
        dev, lib, st = h.device, N.lib(), N.stream(h.device)
        proj = self.in_proj(h)
        code = N.block_dtype_code(proj.dtype)
        cq = torch.empty((T, self.q_rank), dtype=proj.dtype, device=dev)
        pt = attn.page_table
        N.check(lib.cvllm_latent_norm_store(
            N.ptr(proj), proj.stride(0), self.q_off, self.q_rank, self.kv_off, r, R, N.ptr(self.q_norm),
            N.ptr(self.kv_norm), self.eps, N.ptr(self.inv_freq), N.ptr(ctx.positions_i32), N.ptr(ctx.token_slot),
            N.ptr(cq), N.ptr(attn.k_cache), N.ptr(pt), pt.stride(0), int(attn.page_size), N.ptr(attn.bh_seq_lens), T,
            RESERVED_BATCH, code, st), "cvllm_latent_norm_store")
        q = self.uq_proj(cq).view(T, H, D + R)
        q_full = torch.empty((T, H, self.row), dtype=proj.dtype, device=dev)
        # q_abs[h] = q_plain[h] W_uk[h]: [H, T, D] x [H, D, r] into the first r columns of the attention's query rows
        torch.bmm(q[:, :, :D].transpose(0, 1), self.uk, out=q_full[:, :, :r].transpose(0, 1))
        N.check(lib.cvllm_latent_q_rope(N.ptr(q), q.stride(0), H, D, R, N.ptr(self.inv_freq), N.ptr(ctx.positions_i32),
                                        N.ptr(q_full), q_full.stride(0), self.row, r, T, code, st), "cvllm_latent_q_rope")
        o_lat = attn.attend(q_full, flat=False)           # [T, H, r], possibly a view of wider rows
        o = torch.empty((T, H, Dv), dtype=proj.dtype, device=dev)
        torch.bmm(o_lat.transpose(0, 1), self.uv.transpose(1, 2), out=o.transpose(0, 1))
        return self.o_proj(sigmoid_gate(o.view(T, H * Dv), proj[:, self.g_off:]))

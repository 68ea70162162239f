"""Tensor-parallel attention block (fused QKV projection, optional Qwen3 q/k RMSNorm, RoPE, KV cache, O projection).

API of the reference: ``TP_Attn`` (python/triton_dist/layers/nvidia/tp_attn.py:79-324).  The reference calls
flashinfer (RMSNorm, RoPE) and flash-attn; here every step is an own kernel: ``qk_norm_rope_kv`` (fused norm + RoPE +
cache write), ``flash_attn_varlen`` / ``gqa_fwd_batch_decode`` (paged attention), tcgen05 GEMMs, fused collectives.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.distributed as dist

from .. import ops
from ..runtime import get_runtime


class TP_Attn:
    def __init__(self, rank: int = 0, world_size: int = 1, group=None):
        self.rank, self.world_size, self.group = rank, world_size, group
        self.wqkv: Optional[torch.Tensor] = None   # [(Hq + 2 Hkv) * D / W, H]
        self.wo: Optional[torch.Tensor] = None     # [H, Hq * D / W]
        self.q_norm_w = self.k_norm_w = None
        self.ag_ctx = self.rs_ctx = self.ar_ctx = self.gemm_ar_ctx = None
        self.rope_theta, self.eps = 1e6, 1e-6

    def _set_dims(self, hidden, num_q_heads, num_kv_heads, head_dim, rope_theta, eps):
        self.hidden, self.head_dim = hidden, head_dim
        self.q_heads = num_q_heads // self.world_size
        self.kv_heads = max(1, num_kv_heads // self.world_size)
        self.rope_theta, self.eps = rope_theta, eps
        self.scale = 1.0 / math.sqrt(head_dim)

    def _init_parameters(self, attn=None, wq=None, wk=None, wv=None, wo=None, q_norm=None, k_norm=None, hidden=None,
                         num_q_heads=None, num_kv_heads=None, head_dim=None, rope_theta=1e6, eps=1e-6, device=None):
        """Shard full q/k/v weights by heads (column parallel) and o by input columns (row parallel)."""
        if attn is not None:
            wq, wk, wv, wo = (attn.q_proj.weight.detach(), attn.k_proj.weight.detach(), attn.v_proj.weight.detach(),
                              attn.o_proj.weight.detach())
            q_norm = getattr(getattr(attn, "q_norm", None), "weight", None)
            k_norm = getattr(getattr(attn, "k_norm", None), "weight", None)
        device = device or get_runtime().device
        self._set_dims(hidden, num_q_heads, num_kv_heads, head_dim, rope_theta, eps)
        W, r, D = self.world_size, self.rank, head_dim
        q = wq[r * self.q_heads * D:(r + 1) * self.q_heads * D]
        if num_kv_heads >= W:
            k = wk[r * self.kv_heads * D:(r + 1) * self.kv_heads * D]
            v = wv[r * self.kv_heads * D:(r + 1) * self.kv_heads * D]
        else:   # fewer KV heads than ranks: replicate the head this rank's query heads use
            kvh = r * num_kv_heads // W
            k, v = wk[kvh * D:(kvh + 1) * D], wv[kvh * D:(kvh + 1) * D]
        self.wqkv = torch.cat([q, k, v], dim=0).to(device).contiguous()
        self.wo = wo[:, r * self.q_heads * D:(r + 1) * self.q_heads * D].to(device).contiguous()
        self.q_norm_w = q_norm.detach().to(device).contiguous() if q_norm is not None else None
        self.k_norm_w = k_norm.detach().to(device).contiguous() if k_norm is not None else None

    def init_random(self, hidden, num_q_heads, num_kv_heads, head_dim, qk_norm=True, rope_theta=1e6, eps=1e-6,
                    dtype=torch.bfloat16, device=None, std=0.02, seed=0):
        device = device or get_runtime().device
        self._set_dims(hidden, num_q_heads, num_kv_heads, head_dim, rope_theta, eps)
        g = torch.Generator(device=device).manual_seed(seed + 104729 * self.rank)
        n_qkv = (self.q_heads + 2 * self.kv_heads) * head_dim
        self.wqkv = (torch.randn(n_qkv, hidden, device=device, generator=g) * std).to(dtype)
        self.wo = (torch.randn(hidden, self.q_heads * head_dim, device=device, generator=g) * std).to(dtype)
        if qk_norm:
            self.q_norm_w = torch.ones(head_dim, device=device, dtype=dtype)
            self.k_norm_w = torch.ones(head_dim, device=device, dtype=dtype)

    # -- contexts -------------------------------------------------------------------------------------------
    def _init_ctx(self, max_M: int, **kw):
        self.ag_ctx = ops.create_ag_gemm_context(max_M=max_M, K=self.hidden, dtype=self.wqkv.dtype)
        self.rs_ctx = ops.create_gemm_rs_context(max_M=max_M, N=self.hidden, output_dtype=self.wqkv.dtype)

    def _init_AR_ctx(self, max_M: int, **kw):
        self.ar_ctx = ops.create_allreduce_ctx(max(4 * max_M * self.hidden * 2, 1 << 20))

    def _init_gemm_ar_ctx(self, max_M: int, **kw):
        self.gemm_ar_ctx = ops.create_gemm_ar_context(max_M=max_M, N=self.hidden, dtype=self.wqkv.dtype)

    def finalize(self):
        for c in (self.ag_ctx, self.rs_ctx, self.ar_ctx, self.gemm_ar_ctx):
            if c is not None:
                c.finalize()
        self.ag_ctx = self.rs_ctx = self.ar_ctx = self.gemm_ar_ctx = None

    # -- core -----------------------------------------------------------------------------------------------
    def _attend(self, qkv: torch.Tensor, position_ids: torch.Tensor, kv_cache, layer_idx: int, bsz: int, q_len: int):
        """qkv [bsz*q_len, (Hq+2Hkv)*D] -> attention output [bsz*q_len, Hq*D]; writes K/V into the cache."""
        k_cache, v_cache = kv_cache.layer(layer_idx)
        slots, kv_lens = kv_cache.step_values(position_ids, bsz, q_len)
        pos = position_ids.reshape(-1).to(torch.int64)
        q = ops.qk_norm_rope_kv(qkv, self.q_norm_w, self.k_norm_w, pos, slots, k_cache, v_cache, self.q_heads,
                                self.kv_heads, self.head_dim, self.eps, self.rope_theta)
        if q_len == 1:
            out = ops.gqa_fwd_batch_decode(q, k_cache, v_cache, kv_cache.decode_workspace(self.q_heads, self.head_dim),
                                           None, kv_lens, kv_cache.block_table, scale=self.scale,
                                           kv_split=kv_cache.kv_splits)
        else:
            cu = kv_cache.cu_seqlens(bsz, q_len)
            out = ops.flash_attn_varlen(q, k_cache, v_cache, kv_cache.block_table, cu, kv_lens, q_len, causal=True,
                                        scale=self.scale)
        return out.reshape(bsz * q_len, self.q_heads * self.head_dim)

    def torch_fwd(self, x: torch.Tensor, position_ids: torch.Tensor, kv_cache, layer_idx: int) -> torch.Tensor:
        """Golden path: cuBLAS projections + NCCL all-reduce around the same attention core.  x [B, S, H]."""
        bsz, q_len, _ = x.shape
        qkv = torch.matmul(x.reshape(bsz * q_len, -1), self.wqkv.t())
        o = self._attend(qkv, position_ids, kv_cache, layer_idx, bsz, q_len)
        o = torch.matmul(o, self.wo.t())
        if self.world_size > 1:
            dist.all_reduce(o, group=self.group)
        return o.reshape(bsz, q_len, -1)

    def dist_triton_fwd(self, x: torch.Tensor, position_ids: torch.Tensor, kv_cache, layer_idx: int) -> torch.Tensor:
        """AG-GEMM (QKV) -> attention -> GEMM-RS (O).  x [B/W, S, H] sharded over the batch dimension."""
        bl, q_len, _ = x.shape
        bsz = bl * self.world_size
        qkv = ops.ag_gemm(x.reshape(bl * q_len, -1), self.wqkv, self.ag_ctx)
        o = self._attend(qkv, position_ids, kv_cache, layer_idx, bsz, q_len)
        o = ops.gemm_rs(o, self.wo, self.rs_ctx)
        return o.reshape(bl, q_len, -1)

    def dist_triton_AR_fwd(self, x: torch.Tensor, position_ids: torch.Tensor, kv_cache, layer_idx: int) -> torch.Tensor:
        bsz, q_len, _ = x.shape
        qkv = ops.gemm(x.reshape(bsz * q_len, -1), self.wqkv)
        o = self._attend(qkv, position_ids, kv_cache, layer_idx, bsz, q_len)
        o = ops.gemm(o, self.wo)
        if self.world_size > 1:
            o = ops.all_reduce(o, ctx=self.ar_ctx)
        return o.reshape(bsz, q_len, -1)

    def dist_triton_gemm_ar_fwd(self, x: torch.Tensor, position_ids: torch.Tensor, kv_cache, layer_idx: int) -> torch.Tensor:
        bsz, q_len, _ = x.shape
        qkv = ops.gemm(x.reshape(bsz * q_len, -1), self.wqkv)
        o = self._attend(qkv, position_ids, kv_cache, layer_idx, bsz, q_len)
        o = ops.gemm_allreduce_op(self.gemm_ar_ctx, o, self.wo)
        return o.reshape(bsz, q_len, -1)

    def set_fwd(self, mode: str = "torch"):
        self.fwd = {"torch": self.torch_fwd, "triton_dist": self.dist_triton_fwd, "ag_rs": self.dist_triton_fwd,
                    "triton_dist_AR": self.dist_triton_AR_fwd, "allreduce": self.dist_triton_AR_fwd,
                    "triton_dist_gemm_ar": self.dist_triton_gemm_ar_fwd, "gemm_ar": self.dist_triton_gemm_ar_fwd}[mode]

    def __call__(self, x, position_ids, kv_cache, layer_idx):
        return self.fwd(x, position_ids, kv_cache, layer_idx)

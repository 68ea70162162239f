"""Ulysses sequence parallelism: QKV projection -> sequence-to-head all-to-all, and head-to-sequence all-to-all -> O
projection.

API of the reference: ``SpUlysessQKVGemmAll2AllKernel`` (kernels/nvidia/sp_ulysess_qkv_gemm_all2all.py:447-844,
``forward`` / ``pre_attn_a2a``) and ``SpUlysessOAll2AllGemmKernel`` (sp_ulysess_o_all2all_gemm.py:395-703,
``forward`` / ``post_attn_a2a``).  The projections run on the tcgen05 GEMM, the exchanges on the peer-store all-to-all
kernel of this package (``csrc/ep_a2a.cu`` ``a2a_single_kernel``): every rank pushes each destination's head slice
straight into that rank's receive buffer and the kernel returns when all sources have arrived.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..runtime import get_runtime


class SpUlysessQKVGemmAll2AllKernel:
    def __init__(self, world_group=None, nnodes: int = 1, sp_size: Optional[int] = None, max_batch_size: int = 1,
                 num_head: int = 32, max_seqlen: int = 4096, head_dim: int = 128, max_num_comm_buf: int = 1,
                 input_dtype: torch.dtype = torch.bfloat16, output_dtype: torch.dtype = torch.bfloat16, **kw):
        rt = get_runtime()
        self.rt = rt
        self.W = rt.world_size if sp_size is None else sp_size
        self.num_head, self.head_dim = num_head, head_dim
        rows = max_batch_size * max_seqlen
        self.a2a_ctx = ops.create_all_to_all_single_2d_context(rows, 3 * (num_head // self.W) * head_dim, output_dtype)

    def pre_attn_a2a(self, qkv_local: torch.Tensor) -> torch.Tensor:
        """[s_local, 3, heads, D] on every rank -> [s_local * W, 3, heads / W, D] (all positions, this rank's heads)."""
        W = self.W
        s_local = qkv_local.shape[0]
        hl = self.num_head // W
        if W == 1:
            return qkv_local
        # destination-major rows: block d holds this rank's positions restricted to rank d's heads
        x = qkv_local.reshape(s_local, 3, W, hl, self.head_dim).permute(2, 0, 1, 3, 4).contiguous()
        x = x.reshape(W * s_local, 3 * hl * self.head_dim)
        y = ops.all_to_all_single_2d(self.a2a_ctx, x, [s_local] * W, [s_local] * W)
        return y.reshape(W * s_local, 3, hl, self.head_dim)

    def forward(self, inputs: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        """inputs [s_local, H], weight [3 * heads * D, H] -> [S, 3, heads / W, D]."""
        qkv = ops.gemm(inputs, weight)
        if bias is not None:
            qkv = qkv + bias
        return self.pre_attn_a2a(qkv.reshape(inputs.shape[0], 3, self.num_head, self.head_dim))

    qkv_pack_a2a = pre_attn_a2a


class SpUlysessOAll2AllGemmKernel:
    def __init__(self, world_group=None, nnodes: int = 1, sp_size: Optional[int] = None, max_batch_size: int = 1,
                 num_head: int = 32, max_seqlen: int = 4096, head_dim: int = 128, input_dtype: torch.dtype = torch.bfloat16,
                 output_dtype: torch.dtype = torch.bfloat16, **kw):
        rt = get_runtime()
        self.rt = rt
        self.W = rt.world_size if sp_size is None else sp_size
        self.num_head, self.head_dim = num_head, head_dim
        rows = max_batch_size * max_seqlen
        self.a2a_ctx = ops.create_all_to_all_single_2d_context(rows, (num_head // self.W) * head_dim, output_dtype)

    def post_attn_a2a(self, attn_out: torch.Tensor) -> torch.Tensor:
        """[S, heads / W, D] (all positions, local heads) -> [s_local, heads, D] (local positions, all heads)."""
        W = self.W
        if W == 1:
            return attn_out
        S = attn_out.shape[0]
        s_local = S // W
        hl = self.num_head // W
        x = attn_out.reshape(S, hl * self.head_dim).contiguous()      # rows already ordered by destination rank
        y = ops.all_to_all_single_2d(self.a2a_ctx, x, [s_local] * W, [s_local] * W)   # [W(src heads), s_local, hl*D]
        return y.reshape(W, s_local, hl, self.head_dim).permute(1, 0, 2, 3).reshape(s_local, self.num_head, self.head_dim)

    def forward(self, inputs: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        """inputs [S, heads / W, D], weight [H, heads * D] -> [s_local, H]."""
        x = self.post_attn_a2a(inputs)
        out = ops.gemm(x.reshape(x.shape[0], -1).contiguous(), weight)
        if bias is not None:
            out = out + bias
        return out

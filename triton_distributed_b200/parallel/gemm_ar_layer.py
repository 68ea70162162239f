"""Thin layer objects over the fused ops, as in the reference: ``GemmARLayer``
(python/triton_dist/layers/nvidia/gemm_allreduce_layer.py:32-116) and ``AllGatherLayer``
(low_latency_allgather_layer.py:30-187)."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..runtime import get_runtime


class GemmARLayer:
    """Row-parallel linear followed by an all-reduce, one launch for decode sizes."""

    def __init__(self, tp_group=None, max_M: int = 256, N: int = 0, K: int = 0, input_dtype: torch.dtype = torch.bfloat16,
                 output_dtype: torch.dtype = torch.bfloat16, local_world_size: int = 8, persistent: bool = True,
                 use_ll_kernel: bool = True, copy_to_local: bool = True, NUM_COMM_SMS: int = 16, **kw):
        self.ctx = ops.create_gemm_ar_context(max_M=max_M, N=N, dtype=output_dtype)

    def forward(self, x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        out = ops.gemm_allreduce_op(self.ctx, x, weight)
        return out if bias is None else out + bias

    __call__ = forward

    def finalize(self):
        self.ctx.finalize()


class AllGatherLayer:
    """Low-latency all-gather of small tensors (``forward_push_2d_ll`` and friends map onto the packet kernel)."""

    def __init__(self, nnodes: int = 1, world_size: Optional[int] = None, rank: Optional[int] = None,
                 max_buffer_size: int = 64 * 1024 * 1024, stages: int = 2):
        rt = get_runtime()
        self.ctx = ops.create_fast_allgather_context(rank, 0, world_size, nnodes, max_buffer_size)

    def forward_push_2d_ll(self, x: torch.Tensor) -> torch.Tensor:
        return ops.all_gather_ll(x, self.ctx)

    forward_push_2d = forward_push_3d = forward_pull = forward_push_2d_ll_multimem = forward_push_2d_ll

    def forward(self, symm_buffer: torch.Tensor) -> torch.Tensor:
        return ops.fast_allgather(symm_buffer, self.ctx)

    def finalize(self):
        self.ctx.finalize()

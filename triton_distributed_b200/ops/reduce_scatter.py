"""Reduce-scatter over rows: ``[M, N]`` per rank -> this rank's ``[M/W, N]`` block of the sum.

API of the reference: ``create_reduce_scater_2d_ctx`` / ``reduce_scatter_2d_op`` / ``ring_reduce``
(python/triton_dist/kernels/nvidia/reduce_scatter.py:148, :857, :815).  The GPU kernel is the
reduce-scatter half of the two-shot all-reduce (peer stores, or NVLS ``multimem.ld_reduce`` of the own
shard); the hierarchical / ring variants of the reference are unnecessary on one NVSwitch domain.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import _native
from ..runtime import Runtime, get_runtime
from .allreduce import MAX_CTAS, _ctas_for
from .common import new_ctx_dev, ref_reduce_scatter


@dataclass
class ReduceScatter2DContext:
    rt: Runtime
    max_M: int
    N: int
    rank: int
    world_size: int
    dtype: torch.dtype
    workspace: Optional[torch.Tensor] = None
    flags: Optional[torch.Tensor] = None
    ctx_dev: Optional[torch.Tensor] = None
    use_nvls: bool = True

    def finalize(self):
        if self.workspace is not None:
            self.rt.symm_free(self.workspace)
            self.rt.symm_free(self.flags)
            self.workspace = None


def create_reduce_scater_2d_ctx(max_M: int, N: int, rank: Optional[int] = None, world_size: Optional[int] = None,
                                local_world_size: Optional[int] = None, dtype: torch.dtype = torch.bfloat16,
                                overlap_with_gemm: bool = True, num_reduction_sms: int = 15) -> ReduceScatter2DContext:
    rt = get_runtime()
    rank = rt.rank if rank is None else rank
    world_size = rt.world_size if world_size is None else world_size
    ctx = ReduceScatter2DContext(rt=rt, max_M=max_M, N=N, rank=rank, world_size=world_size, dtype=dtype)
    if rt.is_cuda and world_size > 1:
        esz = torch.empty((), dtype=dtype).element_size()
        msg = (max_M * N * esz + 16 * world_size - 1) // (16 * world_size) * (16 * world_size)
        ctx.workspace = rt.symm_tensor((2 * 2 * msg + 1024,), torch.uint8, zero=False)
        ctx.flags = rt.symm_tensor((2, 2, world_size, MAX_CTAS), torch.int32)
        ctx.ctx_dev = new_ctx_dev(rt)
        torch.cuda.synchronize()
        rt.host_barrier()
    return ctx


create_reduce_scatter_2d_ctx = create_reduce_scater_2d_ctx


def ring_reduce(slots: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Sum over the leading (source-rank) dimension in fp32: ``[W, m, N] -> [m, N]``."""
    res = slots.float().sum(dim=0).to(slots.dtype)
    if out is not None:
        out.copy_(res)
        return out
    return res


def reduce_scatter_2d_op(input: torch.Tensor, ctx: ReduceScatter2DContext,
                         output: Optional[torch.Tensor] = None) -> torch.Tensor:
    rt = ctx.rt
    W = ctx.world_size
    if (not _native.use_native(input)) or W == 1 or input.dtype not in (torch.bfloat16, torch.float16, torch.float32):
        res = ref_reduce_scatter(input, rt.group)
        if output is not None:
            output.copy_(res)
            return output
        return res
    lib = _native.load(True)
    x = input.contiguous()
    M, N = x.shape
    if M % W != 0:
        raise ValueError("reduce_scatter: rows must be divisible by the world size")
    nbytes = x.numel() * x.element_size()
    if (nbytes // W) % 16 != 0:
        raise ValueError("reduce_scatter: the per-rank block must be a multiple of 16 bytes")
    if output is None:
        output = torch.empty((M // W, N), dtype=x.dtype, device=x.device)
    method = 3 if (ctx.use_nvls and rt.has_multicast) else 1
    lib.all_reduce(rt.heap, x.view(-1), output.view(-1), ctx.workspace, ctx.flags, ctx.ctx_dev, method, True, MAX_CTAS,
                   _ctas_for(nbytes // W, x.device), rt.config.wait_timeout_s)
    return output

"""``all_to_all_single`` with uneven splits over the symmetric heap.

API of the reference: ``create_all_to_all_single_2d_context`` / ``all_to_all_single_2d``
(kernels/nvidia/all_to_all_single_2d.py:99-171).  The split matrix is exchanged with the low-latency packet
all-gather, then one kernel stores every destination's rows at their final offsets and waits for all sources.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from .. import _native
from ..runtime import Runtime, get_runtime
from .allgather import all_gather_ll, create_fast_allgather_context
from .common import new_ctx_dev, ref_all_to_all_single


@dataclass
class AllToAllSingle2DContext:
    rt: Runtime
    max_rows: int
    row_elems: int
    dtype: torch.dtype
    out: Optional[torch.Tensor] = None
    flags: Optional[torch.Tensor] = None
    ctx_dev: Optional[torch.Tensor] = None
    ag_ctx: object = None
    calls: int = 0

    def finalize(self):
        if self.out is not None:
            self.rt.symm_free(self.out)
            self.rt.symm_free(self.flags)
            self.out = None
        if self.ag_ctx is not None:
            self.ag_ctx.finalize()


def create_all_to_all_single_2d_context(max_rows: int, row_elems: int, dtype: torch.dtype = torch.bfloat16
                                        ) -> AllToAllSingle2DContext:
    """``max_rows`` = most rows any rank can receive in one call."""
    rt = get_runtime()
    ctx = AllToAllSingle2DContext(rt, max_rows, row_elems, dtype)
    if rt.is_cuda and rt.world_size > 1:
        ctx.out = rt.symm_tensor((2, max_rows, row_elems), dtype, zero=False)   # alternating by call parity
        ctx.flags = rt.symm_tensor((rt.world_size,), torch.int32)
        ctx.ctx_dev = new_ctx_dev(rt)
        ctx.ag_ctx = create_fast_allgather_context(max_ll_bytes=64 * 1024)
        torch.cuda.synchronize()
        rt.host_barrier()
    return ctx


def all_to_all_single_2d(ctx: AllToAllSingle2DContext, input: torch.Tensor, output_splits: Optional[List[int]] = None,
                         input_splits: Optional[List[int]] = None) -> torch.Tensor:
    """Rows ``input_splits[d]`` of ``input`` go to rank d; returns the received rows ordered by source rank."""
    rt = ctx.rt
    W = rt.world_size
    if W == 1 or not _native.use_native(input):
        return ref_all_to_all_single(input, output_splits, input_splits, rt.group)
    lib = _native.load(True)
    if input_splits is None:
        input_splits = [input.shape[0] // W] * W
    sp = torch.tensor(input_splits, dtype=torch.int32, device=input.device)
    splits_all = all_gather_ll(sp, ctx.ag_ctx).contiguous()            # [W src][W dst]
    n_out = sum(output_splits) if output_splits is not None else int(splits_all[:, rt.rank].sum().item())
    if n_out > ctx.max_rows:
        raise ValueError("all_to_all_single_2d: more rows than the context was created for")
    x = input.contiguous()
    if (x.shape[1] * x.element_size()) % 16 != 0:
        raise ValueError("all_to_all_single_2d: rows must be a multiple of 16 bytes")
    # two receive buffers alternate (a peer may start its next call while this rank still copies the result out)
    buf = ctx.out[ctx.calls & 1]
    ctx.calls += 1
    lib.a2a_single(rt.heap, x, buf, splits_all, ctx.flags, ctx.ctx_dev, 4, rt.config.wait_timeout_s)
    return buf[:n_out].clone()

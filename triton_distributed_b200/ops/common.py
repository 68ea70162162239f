"""Shared helpers of the op wrappers: per-context device state and torch reference collectives."""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from ..runtime import Runtime, get_runtime


def new_ctx_dev(rt: Runtime) -> torch.Tensor:
    """Device-side call state of a fused-op context: [epoch, done counter, grid barrier word, pad...]."""
    t = torch.zeros(8, dtype=torch.int32, device=rt.device)
    t[0] = 1  # epochs start at 1 so that zero-initialised flags mean "nothing arrived"
    return t


def poison_unused_parity(buf: torch.Tensor, calls: int) -> None:
    """Debug aid (``TDB200_DEBUG=1``): ``buf`` is a double-buffered heap object ``[2, ...]`` whose half ``epoch & 1`` the
    call with epoch ``calls + 1`` uses.  Fill the OTHER half with NaN (0xFF bytes for integer / fp8 data) before the
    launch, in stream order.  That half was last written for the previous call, which this rank has finished, and no
    peer can write it again before this rank's launch of the current call has pushed its data (a peer's next call
    needs them), so the fill races with nothing; a kernel that reads a stale or wrong-parity tile then produces NaN
    instead of plausible numbers.  Eager mode only: under CUDA-graph replay the host's call count is not the epoch."""
    half = buf[(calls + 1) & 1 ^ 1]
    if half.dtype.is_floating_point and half.element_size() >= 2:
        half.fill_(float("nan"))
    else:
        half.view(torch.uint8).fill_(0xFF)


def sm_count(device) -> int:
    return torch.cuda.get_device_properties(device).multi_processor_count


# ---------------------------------------------------------------------- torch reference collectives
# They work on any backend torch.distributed offers (gloo on CPU, NCCL on GPU) and are both the
# baseline the fused kernels are compared with and the CPU backend of every op.

def ref_all_gather(x: torch.Tensor, group=None) -> torch.Tensor:
    rt = get_runtime()
    group = group if group is not None else rt.group
    W = dist.get_world_size(group)
    if W == 1:
        return x.clone()
    out = torch.empty((W * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x.contiguous(), group=group)
    return out


def ref_all_reduce(x: torch.Tensor, group=None) -> torch.Tensor:
    rt = get_runtime()
    group = group if group is not None else rt.group
    y = x.clone()
    if dist.get_world_size(group) > 1:
        dist.all_reduce(y, group=group)
    return y


def ref_reduce_scatter(x: torch.Tensor, group=None) -> torch.Tensor:
    """Sum over ranks, each rank keeps its row block.  gloo has no reduce_scatter: all_reduce + slice there."""
    rt = get_runtime()
    group = group if group is not None else rt.group
    W = dist.get_world_size(group)
    if W == 1:
        return x.clone()
    rank = dist.get_rank(group)
    m = x.shape[0] // W
    if x.is_cuda:
        out = torch.empty((m,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x.contiguous(), group=group)
        return out
    y = x.clone()
    dist.all_reduce(y, group=group)
    return y[rank * m:(rank + 1) * m].clone()


def ref_all_to_all_single(x: torch.Tensor, out_splits: Optional[List[int]], in_splits: Optional[List[int]],
                          group=None) -> torch.Tensor:
    rt = get_runtime()
    group = group if group is not None else rt.group
    W = dist.get_world_size(group)
    if W == 1:
        return x.clone()
    n_out = sum(out_splits) if out_splits is not None else x.shape[0]
    out = torch.empty((n_out,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    if x.is_cuda:
        dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=group)
        return out
    # gloo: emulate with all_gather of padded chunks
    in_splits = in_splits or [x.shape[0] // W] * W
    out_splits = out_splits or [x.shape[0] // W] * W
    rank = dist.get_rank(group)
    gathered: List = [None] * W
    dist.all_gather_object(gathered, (x, in_splits), group=group)
    pieces = []
    for src in range(W):
        xs, sp = gathered[src]
        off = sum(sp[:rank])
        pieces.append(xs[off:off + sp[rank]])
    return torch.cat(pieces, dim=0)

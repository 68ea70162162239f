"""All-gather: in-place on a symmetric buffer (push / NVLS / pull) and the low-latency packet variant.

API of the reference: ``AllGatherMethod`` / ``get_auto_all_gather_method`` / ``cp_engine_producer_all_gather_intra_node``
(python/triton_dist/kernels/nvidia/allgather.py:46-263) and ``create_fast_allgather_context`` / ``fast_allgather``
(low_latency_allgather.py:798, :968).  The copy-engine producers of the reference become SM kernels here because
the all-gather that matters for overlap lives inside the GEMM launch (``ag_gemm``); this module is the standalone
collective.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Optional

import torch

from .. import _native
from ..runtime import Runtime, get_runtime
from .allreduce import MAX_CTAS, _ctas_for
from .common import new_ctx_dev, ref_all_gather


class AllGatherMethod(enum.Enum):
    Auto = 0
    All2All_IntraNode = 1      # full-mesh push
    All2All_Pull = 2           # full-mesh pull
    NVLS = 3                   # multimem.st broadcast
    LL = 4                     # in-band flag packets (small messages)
    Ring1D_IntraNode = 5       # kept for API parity: served by the push kernel
    Ring2D_IntraNode = 6


def get_auto_all_gather_method(nbytes_per_rank: int = 0, has_multicast: Optional[bool] = None) -> AllGatherMethod:
    if has_multicast is None:
        try:
            has_multicast = get_runtime().has_multicast
        except RuntimeError:
            has_multicast = False
    if nbytes_per_rank and nbytes_per_rank <= 32 * 1024:
        return AllGatherMethod.LL
    return AllGatherMethod.NVLS if has_multicast else AllGatherMethod.All2All_IntraNode


@dataclass
class FastAllGatherContext:
    rt: Runtime
    rank: int
    num_ranks: int
    max_buffer_size: int
    flags: Optional[torch.Tensor] = None
    ctx_dev: Optional[torch.Tensor] = None
    ll_staging: Optional[torch.Tensor] = None   # heap, uint8 [2][W * 2 * max_ll_bytes]
    ll_ctx_dev: Optional[torch.Tensor] = None
    max_ll_bytes: int = 0

    def finalize(self):
        if self.flags is not None:
            self.rt.symm_free(self.flags)
            self.rt.symm_free(self.ll_staging)
            self.flags = None


def create_fast_allgather_context(rank: Optional[int] = None, node: int = 0, num_ranks: Optional[int] = None,
                                  num_nodes: int = 1, max_buffer_size: int = 64 * 1024 * 1024,
                                  max_ll_bytes: int = 256 * 1024) -> FastAllGatherContext:
    rt = get_runtime()
    rank = rt.rank if rank is None else rank
    num_ranks = rt.world_size if num_ranks is None else num_ranks
    ctx = FastAllGatherContext(rt=rt, rank=rank, num_ranks=num_ranks, max_buffer_size=max_buffer_size,
                               max_ll_bytes=max_ll_bytes)
    if rt.is_cuda and num_ranks > 1:
        ctx.flags = rt.symm_tensor((2, 2, num_ranks, MAX_CTAS), torch.int32)
        ctx.ctx_dev = new_ctx_dev(rt)
        ctx.ll_staging = rt.symm_tensor((2, num_ranks * 2 * max_ll_bytes), torch.uint8)
        ctx.ll_ctx_dev = new_ctx_dev(rt)
        torch.cuda.synchronize()
        rt.host_barrier()
    return ctx


def fast_allgather(symm_buffer: torch.Tensor, ctx: FastAllGatherContext,
                   mode: AllGatherMethod = AllGatherMethod.Auto) -> torch.Tensor:
    """In-place all-gather of a symmetric buffer ``[W * n, ...]``: slot ``rank`` is valid on entry."""
    rt = ctx.rt
    W = ctx.num_ranks
    if W == 1:
        return symm_buffer
    if not _native.use_native(symm_buffer):
        n = symm_buffer.shape[0] // W
        full = ref_all_gather(symm_buffer[ctx.rank * n:(ctx.rank + 1) * n], rt.group)
        symm_buffer.copy_(full)
        return symm_buffer
    lib = _native.load(True)
    if not rt.is_symmetric(symm_buffer):
        raise ValueError("fast_allgather: the buffer must come from the symmetric heap")
    nbytes = symm_buffer.numel() * symm_buffer.element_size()
    shard = nbytes // W
    if shard % 16 != 0:
        raise ValueError("fast_allgather: the per-rank shard must be a multiple of 16 bytes")
    if mode in (AllGatherMethod.Auto, AllGatherMethod.LL):
        mode = AllGatherMethod.NVLS if rt.has_multicast else AllGatherMethod.All2All_IntraNode
    k = {AllGatherMethod.NVLS: 1, AllGatherMethod.All2All_Pull: 2}.get(mode, 0)
    if k == 1 and not rt.has_multicast:
        k = 0
    lib.all_gather(rt.heap, symm_buffer, shard, ctx.flags, ctx.ctx_dev, k, MAX_CTAS, _ctas_for(shard, symm_buffer.device),
                   rt.config.wait_timeout_s)
    return symm_buffer


def all_gather_ll(x: torch.Tensor, ctx: FastAllGatherContext, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Low-latency all-gather of a small local tensor ``x`` -> ``[W, *x.shape]`` (in-band flag packets)."""
    rt = ctx.rt
    W = ctx.num_ranks
    if W == 1:
        return x.unsqueeze(0).clone()
    if not _native.use_native(x):
        return ref_all_gather(x.unsqueeze(0), rt.group)
    lib = _native.load(True)
    x = x.contiguous()
    nbytes = x.numel() * x.element_size()
    if nbytes % 8 != 0 or nbytes > ctx.max_ll_bytes:
        raise ValueError("all_gather_ll: size must be a multiple of 8 bytes and at most max_ll_bytes")
    if out is None:
        out = torch.empty((W,) + tuple(x.shape), dtype=x.dtype, device=x.device)
    lib.all_gather_ll(rt.heap, x, out, ctx.ll_staging, ctx.ll_ctx_dev, max(1, min(16, nbytes // 8192)),
                      rt.config.wait_timeout_s)
    return out


def all_gather(x: torch.Tensor, ctx: Optional[FastAllGatherContext] = None) -> torch.Tensor:
    """Convenience: gather ``x`` [n, ...] from all ranks -> [W*n, ...] using the best method for its size."""
    rt = get_runtime() if ctx is None else ctx.rt
    if rt.world_size == 1 or not _native.use_native(x) or ctx is None:
        return ref_all_gather(x, rt.group)
    nbytes = x.numel() * x.element_size()
    if nbytes <= min(32 * 1024, ctx.max_ll_bytes) and nbytes % 8 == 0:
        return all_gather_ll(x, ctx).reshape((rt.world_size * x.shape[0],) + tuple(x.shape[1:]))
    buf = rt.symm_tensor((rt.world_size,) + tuple(x.shape), x.dtype, zero=False)
    buf[rt.rank].copy_(x)
    fast_allgather(buf, ctx)
    res = buf.reshape((rt.world_size * x.shape[0],) + tuple(x.shape[1:])).clone()
    rt.symm_free(buf)
    return res


def cp_engine_producer_all_gather_intra_node(rank, num_ranks, local_tensor, remote_buffers, ag_stream=None,
                                             signal_buffers=None, all_gather_method=AllGatherMethod.Auto):
    """Copy-engine all-gather: copies every peer's shard into the local buffer with ``cudaMemcpyAsync``
    (``Tensor.copy_`` between peer-mapped views) on ``ag_stream`` and then raises the shard's flag with a
    stream write - the reference's full-mesh pull (allgather.py:106-137)."""
    rt = get_runtime()
    lib = _native.load(True)
    stream = ag_stream or torch.cuda.current_stream()
    n = local_tensor.shape[0]
    with torch.cuda.stream(stream):
        for i in range(1, num_ranks):
            src = (rank + i) % num_ranks
            remote_buffers[rank][src * n:(src + 1) * n].copy_(remote_buffers[src][src * n:(src + 1) * n], non_blocking=True)
            if signal_buffers is not None:
                lib.stream_write_value32(signal_buffers[rank][src:src + 1].data_ptr(), 1)


def cp_engine_producer_all_gather_inter_node(rank, num_ranks, local_tensor, remote_buffers, ag_stream=None,
                                             signal_buffers=None, all_gather_method=AllGatherMethod.Auto,
                                             internode_ag_stream=None, local_world_size=None):
    """The reference's two-level producer (allgather.py:539: peers of the same node by copy engine, other nodes over the
    network).  One NVSwitch domain has no second level, so every peer is a same-node peer and the copies are those of
    :func:`cp_engine_producer_all_gather_intra_node`; ``internode_ag_stream`` and ``local_world_size`` are accepted for
    signature compatibility."""
    return cp_engine_producer_all_gather_intra_node(rank, num_ranks, local_tensor, remote_buffers, ag_stream,
                                                    signal_buffers, all_gather_method)

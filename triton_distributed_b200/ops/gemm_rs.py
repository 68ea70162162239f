"""GEMM -> ReduceScatter in one kernel launch (``gemm_rs``).

API of the reference: ``create_gemm_rs_context`` / ``gemm_rs``
(python/triton_dist/kernels/nvidia/gemm_reduce_scatter.py:70, :569).  Inputs: ``a`` [M, K/W], ``b`` [N, K/W]
(row-parallel weight, K-major); output [M/W, N] = this rank's row block of ``sum_r a_r @ b_r^T``.

GPU path: ``csrc/gemm_sm100.cu`` in reduce-scatter mode - the tcgen05 epilogue stores every partial tile
straight into the owner rank's slot over NVLink (the reference's ``fuse_scatter``) with a per-tile epoch
flag.  Tiles are visited starting with the next rank's rows, so the own rows come last; in the CTA-pair kernel
their epilogue adds the partials that have arrived from the other ranks to the fp32 accumulators and writes the
output, in the single-CTA kernel all CTAs reduce the arrived slots of the local row block after their last tile.
CPU / reference path: ``matmul`` + ``reduce_scatter_tensor`` (layers/nvidia/tp_mlp.py:254-265).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import _native
from ..runtime import Runtime, get_runtime
from ..utils.oplog import logged_op
from .gemm import use_cta_pair
from .common import new_ctx_dev, ref_reduce_scatter, sm_count

BLOCK_M = 128


@dataclass
class GEMMReduceScatterTensorParallelContext:
    rt: Runtime
    rank: int
    world_size: int
    max_M: int
    N: int
    output_dtype: torch.dtype
    BLOCK_N: int = 256
    kernel_form: str = "auto"   # "auto" | "single" (128 x BLOCK_N tiles) | "pair" (256 x 256 tiles over two SMs)
    num_ctas: int = 0
    slots: Optional[torch.Tensor] = None   # heap [2][W][max_M/W][N]
    flags: Optional[torch.Tensor] = None   # heap [2][W][max_tiles]
    ctx_dev: Optional[torch.Tensor] = None
    max_tiles: int = 0
    calls: int = 0
    stats: Optional[torch.Tensor] = None   # optional int64 [num_ctas, 8] stall counters filled by the pair kernel

    @property
    def max_seg_rows(self) -> int:
        return self.max_M // self.world_size

    def finalize(self):
        if self.slots is not None:
            self.rt.symm_free(self.slots)
            self.rt.symm_free(self.flags)
            self.slots = None
            self.flags = None


def create_gemm_rs_context(max_M: int, N: int, rank: Optional[int] = None, world_size: Optional[int] = None,
                           local_world_size: Optional[int] = None, output_dtype: torch.dtype = torch.bfloat16,
                           rs_stream=None, BLOCK_M: int = 128, BLOCK_N: int = 256, BLOCK_K: int = 64,
                           GROUP_M: int = 8, stages: int = 3) -> GEMMReduceScatterTensorParallelContext:
    """Allocate the per-source slots and tile flags (collective call)."""
    rt = get_runtime()
    rank = rt.rank if rank is None else rank
    world_size = rt.world_size if world_size is None else world_size
    max_M = (max_M + world_size - 1) // world_size * world_size
    ctx = GEMMReduceScatterTensorParallelContext(rt=rt, rank=rank, world_size=world_size, max_M=max_M, N=N,
                                                 output_dtype=output_dtype,
                                                 BLOCK_N=BLOCK_N if BLOCK_N in (128, 256) else 256)
    if rt.is_cuda and world_size > 1:
        seg = ctx.max_seg_rows
        ctx.max_tiles = ((seg + BLOCK_M - 1) // BLOCK_M) * ((N + 127) // 128)
        ctx.slots = rt.symm_tensor((2, world_size, seg, N), output_dtype, zero=False)
        ctx.flags = rt.symm_tensor((2, world_size, ctx.max_tiles), torch.int32)
        ctx.ctx_dev = new_ctx_dev(rt)
        torch.cuda.synchronize()
        rt.host_barrier()
    return ctx


def gemm_rs_reference(a: torch.Tensor, b: torch.Tensor, group=None) -> torch.Tensor:
    """reduce_scatter(a @ b^T) with torch.matmul + torch.distributed."""
    return ref_reduce_scatter(torch.matmul(a, b.t()), group)


def _rs_meta(a, b, ctx, *args, **kw):
    W = ctx.world_size
    M, K = a.shape
    N = b.shape[0]
    return {"shape": {"M": M, "N": N, "K": K * W, "world": W}, "flops": 2.0 * M * N * K,
            "link_bytes": (W - 1) / max(W, 1) * M * N * a.element_size()}


@logged_op("gemm_rs", _rs_meta)
def gemm_rs(a: torch.Tensor, b: torch.Tensor, ctx: GEMMReduceScatterTensorParallelContext, persistent: bool = True,
            fuse_scatter: bool = True, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a`` [M, K_local], ``b`` [N, K_local] -> [M/W, N]."""
    rt = ctx.rt
    if not _native.use_native(a, b) or a.dtype != torch.bfloat16:
        res = gemm_rs_reference(a, b, rt.group)
        if out is not None:
            out.copy_(res)
            return out
        return res
    lib = _native.load(True)
    W = ctx.world_size
    if W == 1:
        from .gemm import gemm
        return gemm(a, b, out=out)
    if a.stride(-1) != 1:
        a = a.contiguous()
    if b.stride(-1) != 1:
        b = b.contiguous()
    M, _ = a.shape
    N = b.shape[0]
    if N != ctx.N:
        raise ValueError(f"gemm_rs: N={N} differs from the context's N={ctx.N}")
    if M % W != 0:
        raise ValueError("gemm_rs: M must be divisible by the world size")
    if out is None:
        out = torch.empty((M // W, N), dtype=a.dtype, device=a.device)
    pair = use_cta_pair(ctx.kernel_form, M // W, N, out)
    if rt.config.debug:
        from .common import poison_unused_parity
        poison_unused_parity(ctx.slots, ctx.calls)
    lib.gemm_rs_bf16(rt.heap, a, b, out, ctx.slots, ctx.flags, ctx.ctx_dev, ctx.max_seg_rows, ctx.max_tiles,
                     512 if pair else ctx.BLOCK_N, ctx.num_ctas or sm_count(a.device), rt.config.wait_timeout_s, ctx.stats)
    ctx.calls += 1
    return out

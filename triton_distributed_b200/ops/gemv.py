"""Decode GEMV with its layer neighbours fused in (``gemv_fused``): for up to sixteen tokens

    out = [residual +] [all_reduce(] f(x) @ w^T [)],   f = identity | RMSNorm(x) * norm_weight | SiLU(gate) * up

in one launch of ``csrc/gemv.cu``.  With these a decoder layer at decode time is four launches plus attention, where
the reference's layer runs rmsnorm, linear, all-reduce, add and activation kernels one after the other
(python/triton_dist/layers/nvidia/tp_attn.py:160-213, tp_mlp.py:196-229, models/dense.py layer forward).  The
all-reduce follows the protocol of the fused GEMM+AllReduce (kernels/nvidia/gemm_allreduce.py:124-315): partial
results in symmetric memory, per-CTA epoch flags, ``multimem.ld_reduce`` or a push + local sum.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import _native
from ..runtime import Runtime, get_runtime
from .common import new_ctx_dev, sm_count

GEMV_MAX_M = 16    # what the kernel accepts
GEMV_FAST_M = 8    # up to here it beats the tcgen05 weight-streaming kernel (two MMA tiles of tokens are mma.sync-bound)


@dataclass
class GemvARContext:
    rt: Runtime
    rank: int
    world_size: int
    N: int
    m_cap: int = GEMV_MAX_M
    use_multimem: bool = True
    partial: Optional[torch.Tensor] = None   # heap
    flags: Optional[torch.Tensor] = None     # heap [W][max_ctas]
    ctx_dev: Optional[torch.Tensor] = None
    max_ctas: int = 0
    calls: int = 0

    def finalize(self):
        if self.partial is not None:
            self.rt.symm_free(self.partial)
            self.rt.symm_free(self.flags)
            self.partial = None
            self.flags = None


def create_gemv_ar_context(N: int, rt: Optional[Runtime] = None, use_multimem: bool = True,
                           device=None) -> GemvARContext:
    """Symmetric scratch for all-reduced GEMVs with ``N`` output columns (shared by every call with that ``N``:
    consecutive calls alternate two buffers by the call epoch kept on the device)."""
    rt = rt or get_runtime()
    ctx = GemvARContext(rt=rt, rank=rt.rank, world_size=rt.world_size, N=N, use_multimem=use_multimem)
    if rt.world_size > 1 and rt.heap is not None:
        mc = use_multimem and rt.has_multicast
        ctx.max_ctas = sm_count(rt.device)
        ctx.partial = rt.symm_tensor((2, 1 if mc else rt.world_size, ctx.m_cap, N), torch.bfloat16)
        ctx.flags = rt.symm_tensor((rt.world_size, ctx.max_ctas), torch.int32)
        ctx.partial.zero_()
        ctx.flags.zero_()
        ctx.ctx_dev = new_ctx_dev(rt)
        torch.cuda.synchronize()
        rt.host_barrier()
    return ctx


def gemv_reference(x: torch.Tensor, w: torch.Tensor, norm_weight: Optional[torch.Tensor] = None, eps: float = 1e-6,
                   silu_mul: bool = False, residual: Optional[torch.Tensor] = None, group=None,
                   all_reduce: bool = False) -> torch.Tensor:
    """fp32 reference of the fused op (all-reduce through torch.distributed when asked for)."""
    xf = x.float()
    if silu_mul:
        k = w.shape[1]
        xf = torch.nn.functional.silu(xf[..., :k]) * xf[..., k:]
    elif norm_weight is not None:
        xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * norm_weight.float()
    y = xf @ w.float().t()
    if all_reduce:
        import torch.distributed as dist
        dist.all_reduce(y, group=group)
    if residual is not None:
        y = y + residual.float()
    return y.to(x.dtype)


def gemv_supported(M: int, K: int) -> bool:
    """Whether ``M`` tokens with ``K`` input features fit the GEMV kernel (token count and shared-memory staging)."""
    if M < 1 or M > GEMV_MAX_M or K % 8 != 0:
        return False
    mp = 1 if M <= 1 else 2 if M <= 2 else 4 if M <= 4 else 8 if M <= 8 else 16
    return K <= (((200 - 8) * 1024 // mp - 64) // 2) // 8 * 8


def gemv_fused(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None,
               norm_weight: Optional[torch.Tensor] = None, eps: float = 1e-6, silu_mul: bool = False,
               residual: Optional[torch.Tensor] = None, ar_ctx: Optional[GemvARContext] = None) -> torch.Tensor:
    """``x`` [M<=16, K] (or [M, 2K] with ``silu_mul``), ``w`` [N, K] -> [M, N].  ``residual`` may be ``out`` itself.
    With ``ar_ctx`` of a multi-rank runtime the per-rank results are summed over the ranks before the residual."""
    M = x.shape[0]
    N, K = w.shape
    do_ar = ar_ctx is not None and ar_ctx.world_size > 1
    if not (_native.use_native(x, w) and x.dtype == torch.bfloat16 and gemv_supported(M, K)):
        res = gemv_reference(x, w, norm_weight, eps, silu_mul, residual,
                             group=ar_ctx.rt.group if do_ar else None, all_reduce=do_ar)
        if out is not None:
            out.copy_(res)
            return out
        return res
    lib = _native.load(True)
    if out is None:
        out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    if do_ar:
        if N != ar_ctx.N:
            raise ValueError(f"gemv_fused: N={N} differs from the context's N={ar_ctx.N}")
        rt = ar_ctx.rt
        lib.gemv_ar_bf16(rt.heap, x, w, out, norm_weight, float(eps), bool(silu_mul), residual, ar_ctx.partial,
                         ar_ctx.flags, ar_ctx.ctx_dev, ar_ctx.m_cap, ar_ctx.max_ctas, 0,
                         bool(ar_ctx.use_multimem and rt.has_multicast), rt.config.wait_timeout_s)
        ar_ctx.calls += 1
    else:
        lib.gemv_bf16(x, w, out, norm_weight, float(eps), bool(silu_mul), residual, 0)
    return out

"""Single-GPU tcgen05 GEMM: ``C[M,N] = A[M,K] @ B[N,K]^T`` (bf16 in, fp32 accumulate, bf16 out).

B is stored K-major ("weight layout", the same convention the reference uses for its TP layers,
python/triton_dist/kernels/nvidia/allgather_gemm.py:656 ``gemm_persistent``).  On CPU tensors the
torch reference is used.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from .. import _native
from ..utils.oplog import logged_op


SKINNY_M = 128   # up to this many rows the weight-streaming kernel wins
# TDB200_SMALL_M_GEMM=cublas sends plain (unfused) GEMMs of 9..SKINNY_M rows to the library instead of the own
# weight-streaming kernel; a measurement switch, the fused GEMM + all-reduce layers are not affected.
_SMALL_M_LIBRARY = os.environ.get("TDB200_SMALL_M_GEMM", "own") == "cublas"


def use_cta_pair(kernel_form: str, rows: int, n: int, out: Optional[torch.Tensor] = None) -> bool:
    """Whether a GEMM with ``rows`` rows per segment and ``n`` columns runs the CTA-pair kernel (256 x 256 tiles over
    two SMs): ``kernel_form`` "pair" / "single" force it, "auto" takes it for problems of at least one pair tile unless
    ``TDB200_GEMM_PAIR=0``.  The pair kernel stores through TMA, so the output rows must be 16-byte aligned."""
    import os
    if out is not None and (out.stride(0) % 8 != 0 or out.data_ptr() % 16 != 0):
        return False
    if kernel_form == "pair":
        return True
    if kernel_form == "single":
        return False
    return os.environ.get("TDB200_GEMM_PAIR", "1") != "0" and rows >= 256 and n >= 256


def gemm_reference(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """fp32 reference: A @ B^T."""
    return (a.float() @ b.float().t()).to(a.dtype)


STALL_COUNTERS = ("producer_flag_wait", "producer_ring_wait", "mma_operand_wait", "mma_accumulator_wait",
                  "epilogue_accumulator_wait", "epilogue_peer_flag_wait", "epilogue_store_wait", "cta_total")


def new_stall_counters(device, num_ctas: int = 148) -> torch.Tensor:
    """Zeroed ``[num_ctas, 8]`` int64 buffer for the pair kernel's optional stall counters (SM cycles per CTA, columns
    named by ``STALL_COUNTERS``).  Pass it as ``stats=`` to :func:`gemm` or set it as ``ctx.stats`` of an AG-GEMM /
    GEMM-RS context; the kernel adds to it, so zero it between measurements."""
    return torch.zeros(num_ctas, len(STALL_COUNTERS), dtype=torch.int64, device=device)


def summarize_stall_counters(stats: torch.Tensor) -> dict:
    """Mean share of a CTA's lifetime spent in each kind of wait (CTAs that ran), plus the maximum per counter."""
    s = stats.detach().to("cpu").double()
    live = s[:, -1] > 0
    if not bool(live.any()):
        return {}
    s = s[live]
    tot = s[:, -1:].clamp(min=1.0)
    frac = s / tot
    out = {f"{n}_mean_frac": float(frac[:, i].mean()) for i, n in enumerate(STALL_COUNTERS[:-1])}
    out.update({f"{n}_max_frac": float(frac[:, i].max()) for i, n in enumerate(STALL_COUNTERS[:-1])})
    out["cta_total_cycles_max"] = float(s[:, -1].max())
    out["ctas"] = int(live.sum())
    return out


def _gemm_meta(a, b, *args, **kw):
    m = a.numel() // a.shape[-1]
    return {"shape": {"M": m, "N": b.shape[0], "K": a.shape[-1]}, "flops": 2.0 * m * b.shape[0] * a.shape[-1]}


@logged_op("gemm", _gemm_meta)
def gemm(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None, block_n: int = 0,
         num_ctas: int = 0, stats: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a`` [M,K] x ``b`` [N,K] -> [M,N].  bf16 CUDA tensors run the sm_100a kernel."""
    if _native.use_native(a, b) and a.dtype == torch.bfloat16:
        lib = _native.load(True)
        if a.stride(-1) != 1:
            a = a.contiguous()
        if b.stride(-1) != 1:
            b = b.contiguous()
        lead = a.shape[:-1]
        a2 = a.reshape(-1, a.shape[-1])
        if out is None:
            out = torch.empty((a2.shape[0], b.shape[0]), dtype=a.dtype, device=a.device)
        if 0 < a2.shape[0] <= SKINNY_M and block_n == 0 and a2.shape[1] % 8 == 0:
            # decode-size M: stream the weights once - the tensor-core GEMV up to eight rows, the swap-AB stream-K
            # kernel above
            from .gemm_ar import skinny_gemm
            from .gemv import GEMV_FAST_M, gemv_fused, gemv_supported
            o2 = out.view(a2.shape[0], b.shape[0])
            if (a2.shape[0] <= GEMV_FAST_M and gemv_supported(a2.shape[0], a2.shape[1]) and b.stride(0) % 8 == 0
                    and a2.stride(0) % 8 == 0 and a2.data_ptr() % 16 == 0 and b.data_ptr() % 16 == 0):
                gemv_fused(a2, b, out=o2)
            elif _SMALL_M_LIBRARY:
                torch.matmul(a2, b.t(), out=o2)
            else:
                skinny_gemm(a2, b, out=o2)
        else:
            lib.gemm_bf16(a2, b, out.view(a2.shape[0], b.shape[0]), block_n, num_ctas, stats)
        return out.view(*lead, b.shape[0])
    res = torch.matmul(a, b.t())
    if out is not None:
        out.copy_(res)
        return out
    return res


linear = gemm

"""Block-scaled fp8 (e4m3) operands for the tensor-parallel GEMMs: 1 x 128 scales for activations, 128 x 128 scales
for weights (the DeepSeek-V3 recipe the reference's EP path uses for its payloads,
python/triton_dist/kernels/nvidia/low_latency_all_to_all.py:36-118, tutorials/04-deepseek-infer-all2all.py).

What exists: quantisers, de-quantisers and ``gemm_fp8_blockscaled`` / ``ag_gemm_fp8`` as *functional* variants - the
operands travel and rest in fp8 (half the bytes of bf16 over NVLink and in HBM), are de-quantised block by block and
multiplied by the bf16 tcgen05 GEMM.  A native ``tcgen05.mma.kind::f8f6f4`` main loop with per-128-K scale promotion
is not written; the numerics below are what such a kernel has to reproduce.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

BLOCK = 128
FP8_MAX = 448.0


def _fp8_dtype():
    return torch.float8_e4m3fn


def quantize_act_1x128(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``x`` [M, K] -> (fp8 [M, K], fp32 scales [M, K / 128]); K must be a multiple of 128."""
    M, K = x.shape
    assert K % BLOCK == 0, "K must be a multiple of 128"
    xb = x.float().reshape(M, K // BLOCK, BLOCK)
    scale = xb.abs().amax(-1).clamp_min(1e-10) / FP8_MAX
    q = (xb / scale[..., None]).clamp(-FP8_MAX, FP8_MAX).to(_fp8_dtype())
    return q.reshape(M, K), scale


def quantize_weight_128x128(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``w`` [N, K] -> (fp8 [N, K], fp32 scales [ceil(N / 128), K / 128])."""
    N, K = w.shape
    assert K % BLOCK == 0, "K must be a multiple of 128"
    nb = (N + BLOCK - 1) // BLOCK
    wp = torch.zeros(nb * BLOCK, K, dtype=torch.float32, device=w.device)
    wp[:N] = w.float()
    wb = wp.reshape(nb, BLOCK, K // BLOCK, BLOCK)
    scale = wb.abs().amax(dim=(1, 3)).clamp_min(1e-10) / FP8_MAX
    q = (wb / scale[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX).to(_fp8_dtype())
    return q.reshape(nb * BLOCK, K)[:N].contiguous(), scale


def dequantize_act_1x128(q: torch.Tensor, scale: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    M, K = q.shape
    return (q.float().reshape(M, K // BLOCK, BLOCK) * scale[..., None]).reshape(M, K).to(dtype)


def dequantize_weight_128x128(q: torch.Tensor, scale: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    N, K = q.shape
    nb = scale.shape[0]
    qp = torch.zeros(nb * BLOCK, K, dtype=torch.float32, device=q.device)
    qp[:N] = q.float()
    w = qp.reshape(nb, BLOCK, K // BLOCK, BLOCK) * scale[:, None, :, None]
    return w.reshape(nb * BLOCK, K)[:N].to(dtype)


def gemm_fp8_blockscaled_reference(a_q, a_s, b_q, b_s) -> torch.Tensor:
    """fp32 reference with the accumulation order of a block-scaled kernel: one partial product per 128-wide K
    block, scaled by ``a_s[m, kb] * b_s[n / 128, kb]`` and summed in fp32."""
    M, K = a_q.shape
    N = b_q.shape[0]
    kb = K // BLOCK
    a = a_q.float().reshape(M, kb, BLOCK)
    b = b_q.float().reshape(N, kb, BLOCK)
    part = torch.einsum("mkc,nkc->kmn", a, b)                               # [kb, M, N]
    bs = b_s.repeat_interleave(BLOCK, dim=0)[:N]                            # [N, kb]
    return (part * a_s.t()[:, :, None] * bs.t()[:, None, :]).sum(0)


def gemm_fp8_blockscaled(a_q: torch.Tensor, a_s: torch.Tensor, b_q: torch.Tensor, b_s: torch.Tensor,
                         out: Optional[torch.Tensor] = None, out_dtype=torch.bfloat16) -> torch.Tensor:
    """``(a_q, a_s)`` [M, K] with 1 x 128 scales times ``(b_q, b_s)`` [N, K] with 128 x 128 scales -> [M, N]."""
    from .gemm import gemm

    a = dequantize_act_1x128(a_q, a_s, out_dtype)
    b = dequantize_weight_128x128(b_q, b_s, out_dtype)
    return gemm(a, b, out=out)


def ag_gemm_fp8(a_q: torch.Tensor, a_s: torch.Tensor, b_q: torch.Tensor, b_s: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather of fp8 activations and their scales (half the NVLink bytes of the bf16 op) followed by the
    block-scaled GEMM: ``a_q`` [M / W, K] row shard, ``b_q`` [N / W, K] column-parallel weight -> [M, N / W]."""
    from .common import ref_all_gather

    a_all = ref_all_gather(a_q.view(torch.uint8), group).view(_fp8_dtype())
    s_all = ref_all_gather(a_s, group)
    return gemm_fp8_blockscaled(a_all, s_all, b_q, b_s)

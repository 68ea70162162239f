"""Memory-bound decoder ops: RMSNorm (+ fused residual add), SiLU-gated multiply, residual add, fused
QK-RMSNorm + RoPE + KV-cache write, embedding gather, arg-max / top-p sampling.

GPU tensors run the sm_100a kernels in ``csrc/ops.cu``; CPU tensors run the torch restatement below, which is
also the oracle of the GPU tests (same role as the reference's mega_triton_kernel/test/torch_impl_utils.py:41-130).
The reference calls flashinfer for RMSNorm / RoPE (layers/nvidia/tp_attn.py:61-67, :173); here they are own kernels.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _native


# ------------------------------------------------------------------ torch references
def rmsnorm_reference(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y * w.float()).to(x.dtype)


def silu_mul_reference(x: torch.Tensor) -> torch.Tensor:
    i = x.shape[-1] // 2
    g, u = x[..., :i].float(), x[..., i:].float()
    return (torch.nn.functional.silu(g) * u).to(x.dtype)


def rope_cos_sin(positions: torch.Tensor, dim: int, theta: float) -> Tuple[torch.Tensor, torch.Tensor]:
    inv = theta ** (-torch.arange(0, dim // 2, dtype=torch.float32, device=positions.device) * 2.0 / dim)
    ang = positions.float()[:, None] * inv[None, :]
    return ang.cos(), ang.sin()


def apply_rope_reference(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """x [T, H, D], rotate-half convention (HF Llama/Qwen)."""
    d = x.shape[-1]
    cos, sin = rope_cos_sin(positions, d, theta)
    x1, x2 = x[..., : d // 2].float(), x[..., d // 2:].float()
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


def qk_norm_rope_kv_reference(qkv, q_norm_w, k_norm_w, positions, slots, k_cache, v_cache, Hq, Hkv, D, eps, theta):
    T = qkv.shape[0]
    q, k, v = qkv.split([Hq * D, Hkv * D, Hkv * D], dim=-1)
    q = q.reshape(T, Hq, D)
    k = k.reshape(T, Hkv, D)
    v = v.reshape(T, Hkv, D)
    if q_norm_w is not None:
        q = rmsnorm_reference(q, q_norm_w, eps)
    if k_norm_w is not None:
        k = rmsnorm_reference(k, k_norm_w, eps)
    q = apply_rope_reference(q, positions, theta)
    k = apply_rope_reference(k, positions, theta)
    sl = slots if slots is not None else torch.arange(T, device=qkv.device)
    ok = sl >= 0
    k_cache.view(-1, Hkv, D)[sl[ok]] = k[ok]
    v_cache.view(-1, Hkv, D)[sl[ok]] = v[ok]
    return q


# ------------------------------------------------------------------ dispatching wrappers
def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RMSNorm over the last dimension.  With ``residual`` (contiguous, same shape): ``residual += x`` in place
    and the norm is taken of the sum."""
    if _native.use_native(x, w) and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
        return _native.load(True).rmsnorm(x, w, float(eps), residual)
    if residual is not None:
        residual.add_(x)
        x = residual
    return rmsnorm_reference(x, w, eps)


def silu_mul(x: torch.Tensor) -> torch.Tensor:
    """``silu(x[..., :I]) * x[..., I:]`` for the fused gate/up projection output."""
    if _native.use_native(x) and x.dtype == torch.bfloat16 and (x.shape[-1] // 2) % 8 == 0:
        return _native.load(True).silu_mul(x)
    return silu_mul_reference(x)


def residual_add(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    if _native.use_native(a, b) and a.dtype == torch.bfloat16 and a.numel() % 8 == 0 and a.is_contiguous() and b.is_contiguous():
        return _native.load(True).add(a, b)
    return a + b


def qk_norm_rope_kv(qkv: torch.Tensor, q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor],
                    positions: torch.Tensor, slots: Optional[torch.Tensor], k_cache: torch.Tensor, v_cache: torch.Tensor,
                    num_q_heads: int, num_kv_heads: int, head_dim: int, eps: float = 1e-6,
                    rope_theta: float = 1e6) -> torch.Tensor:
    """Packed ``qkv`` [T, (Hq+2Hkv)*D] -> q [T, Hq, D] (RMS-normed per head when a weight is given, rotated);
    k (normed, rotated) and v are written to ``k_cache`` / ``v_cache`` (any shape that flattens to
    [slots, Hkv, D]) at ``slots[t]`` (negative = skip)."""
    if _native.use_native(qkv, k_cache, v_cache) and qkv.dtype == torch.bfloat16:
        return _native.load(True).qk_norm_rope_kv(qkv, q_norm_w, k_norm_w, positions, slots, k_cache, v_cache,
                                                  num_q_heads, num_kv_heads, head_dim, float(eps), float(rope_theta))
    return qk_norm_rope_kv_reference(qkv, q_norm_w, k_norm_w, positions, slots, k_cache, v_cache, num_q_heads,
                                     num_kv_heads, head_dim, eps, rope_theta)


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    if _native.use_native(ids, table) and table.dtype == torch.bfloat16 and table.shape[1] % 8 == 0:
        return _native.load(True).embedding(ids, table)
    return torch.nn.functional.embedding(ids, table)


def argmax(logits: torch.Tensor) -> torch.Tensor:
    if _native.use_native(logits) and logits.dtype == torch.float32 and logits.dim() == 2:
        return _native.load(True).argmax(logits.contiguous())
    return torch.argmax(logits, dim=-1)


def sample_token(logits: torch.Tensor, temperature: float = 0.0, top_p: float = 1.0,
                 generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """Greedy when ``temperature == 0`` (own arg-max kernel); nucleus sampling otherwise (the reference calls
    flashinfer's top-p sampler here, models/utils.py:86)."""
    if temperature <= 0.0:
        return argmax(logits.float())
    probs = torch.softmax(logits.float() / temperature, dim=-1)
    sp, si = torch.sort(probs, dim=-1, descending=True)
    cum = torch.cumsum(sp, dim=-1)
    sp = torch.where(cum - sp > top_p, torch.zeros_like(sp), sp)
    sp = sp / sp.sum(dim=-1, keepdim=True)
    pick = torch.multinomial(sp, 1, generator=generator)
    return si.gather(-1, pick).squeeze(-1)


def abs_sum(x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 sum of |x| (a cheap result checksum that a host can read back in 4 bytes)."""
    if _native.use_native(x) and x.dtype == torch.bfloat16 and x.is_contiguous():
        if out is None:
            out = torch.zeros(1, dtype=torch.float32, device=x.device)
        _native.load(True).abs_sum(x, out)
        return out
    res = x.float().abs().sum().reshape(1)
    if out is not None:
        out.copy_(res)
        return out
    return res

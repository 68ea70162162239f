"""Attention over a paged KV cache: prefill (var-len, causal, GQA), split-KV decode, distributed flash-decode.

API of the reference: ``gqa_fwd_batch_decode`` / ``gqa_fwd_batch_decode_intra_rank`` / ``gqa_fwd_batch_decode_persistent``
(python/triton_dist/kernels/nvidia/flash_decode.py:763, :847, :931) and the flash-attention calls of its layers
(layers/nvidia/tp_attn.py:206).  GPU path: ``csrc/attn.cu``; CPU path and test oracle: the fp32 torch restatement here.

Cache layout: ``[num_pages, page_size, Hkv, D]`` with an int32 ``block_table [B, max_pages]``; a dense per-sequence
cache ``[B, max_len, Hkv, D]`` is the case ``page_size = max_len`` with ``block_table = arange(B)[:, None]``.
"""
from __future__ import annotations

import math
import os
from typing import Optional, Tuple

import torch

from .. import _native


def dense_block_table(batch: int, device) -> torch.Tensor:
    return torch.arange(batch, dtype=torch.int32, device=device).unsqueeze(1).contiguous()


def _gather_kv(k_cache, v_cache, block_table, b: int, n: int):
    """First ``n`` tokens of sequence ``b`` as [n, Hkv, D] (reference path)."""
    page = k_cache.shape[1]
    npages = (n + page - 1) // page
    pages = block_table[b, :npages].long()
    k = k_cache[pages].reshape(-1, k_cache.shape[2], k_cache.shape[3])[:n]
    v = v_cache[pages].reshape(-1, v_cache.shape[2], v_cache.shape[3])[:n]
    return k, v


def attention_reference(q, k_cache, v_cache, block_table, cu_seqlens_q, kv_lens, q_pos0=None, causal=True,
                        scale=None, softcap: float = 0.0, return_lse: bool = False):
    """fp32 softmax attention, one sequence at a time.  q [T, Hq, D] packed by ``cu_seqlens_q``."""
    T, Hq, D = q.shape
    Hkv = k_cache.shape[2]
    g = Hq // Hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    out = torch.zeros_like(q, dtype=torch.float32)
    lse = torch.full((Hq, T), float("-inf"), dtype=torch.float32, device=q.device)
    cu = cu_seqlens_q.tolist()
    for b in range(len(cu) - 1):
        qs, qe = cu[b], cu[b + 1]
        n = int(kv_lens[b])
        if qe == qs or n == 0:
            continue
        k, v = _gather_kv(k_cache, v_cache, block_table, b, n)
        kf = k.float().repeat_interleave(g, dim=1)   # [n, Hq, D]
        vf = v.float().repeat_interleave(g, dim=1)
        s = torch.einsum("qhd,khd->hqk", q[qs:qe].float(), kf) * scale
        if softcap > 0:
            s = softcap * torch.tanh(s / softcap)
        if causal:
            p0 = int(q_pos0[b]) if q_pos0 is not None else n - (qe - qs)
            qpos = torch.arange(qe - qs, device=q.device) + p0
            kpos = torch.arange(n, device=q.device)
            s = s.masked_fill(kpos[None, None, :] > qpos[None, :, None], float("-inf"))
        l = torch.logsumexp(s, dim=-1)
        p = torch.exp(s - l.unsqueeze(-1))
        p = torch.nan_to_num(p, nan=0.0)
        out[qs:qe] = torch.einsum("hqk,khd->qhd", p, vf)
        lse[:, qs:qe] = l
    if return_lse:
        return out.to(q.dtype), lse
    return out.to(q.dtype)


SM100_PREFILL_MIN_Q = 128      # below this the 64-row mma.sync kernel has less padding and no KV packing pass
_PENDING_ERRORS = []            # error flags of tcgen05 prefill launches that have not been looked at yet


def check_attention_errors() -> None:
    """Raise if a bounded wait inside a tcgen05 prefill kernel gave up since the last check (synchronises)."""
    flags, _PENDING_ERRORS[:] = list(_PENDING_ERRORS), []
    codes = [int(f.item()) for f in flags]
    if any(c == 2 for c in codes):
        raise RuntimeError("flash_fwd_sm100: the dynamic shared-memory window was not 1024-byte aligned")
    if any(c != 0 for c in codes):
        raise RuntimeError("flash_fwd_sm100: a wait inside the kernel timed out")


def flash_attn_varlen(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                      cu_seqlens_q: torch.Tensor, kv_lens: torch.Tensor, max_q_len: int,
                      q_pos0: Optional[torch.Tensor] = None, causal: bool = True, scale: Optional[float] = None,
                      softcap: float = 0.0, return_lse: bool = False, max_kv_len: Optional[int] = None,
                      impl: str = "auto"):
    """Prefill / context attention.  ``q`` [T, Hq, D] packed; query row i of sequence b has absolute position
    ``q_pos0[b] + i`` (default: the queries are the last ``q_len`` positions of the ``kv_lens[b]`` visible tokens).

    ``impl``: "auto" picks the tcgen05 kernel (head dim 128, no soft cap, at least ``SM100_PREFILL_MIN_Q`` query rows per
    sequence) and otherwise the ``mma.sync`` kernel; "sm100" / "mma" force one.  ``max_kv_len`` (an upper bound of
    ``kv_lens``) saves the tcgen05 path a device-to-host read."""
    D = q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if _native.use_native(q, k_cache, v_cache) and q.dtype == torch.bfloat16 and D in (64, 128):
        lib = _native.load(True)
        lse = torch.empty((q.shape[1], q.shape[0]), dtype=torch.float32, device=q.device) if return_lse else None
        sm100_ok = D == 128 and softcap == 0.0 and k_cache.dtype == torch.bfloat16 and os.environ.get("TDB200_ATTN_SM100", "1") != "0"
        if impl == "sm100" and not sm100_ok:
            raise ValueError("flash_attn_varlen: the tcgen05 kernel needs head dim 128, bf16 caches and no soft cap")
        if impl == "sm100" or (impl == "auto" and sm100_ok and max_q_len >= SM100_PREFILL_MIN_Q):
            if max_kv_len is None:
                max_kv_len = int(kv_lens.max().item())
            out, err = lib.flash_fwd_sm100(q.contiguous(), k_cache.contiguous(), v_cache.contiguous(), block_table.contiguous(),
                                           cu_seqlens_q, kv_lens, q_pos0, int(max_q_len), max(int(max_kv_len), 1),
                                           bool(causal), float(scale), lse)
            _PENDING_ERRORS.append(err)
            if len(_PENDING_ERRORS) > 64:
                check_attention_errors()
            return (out, lse) if return_lse else out
        out = lib.flash_fwd(q.contiguous(), k_cache, v_cache, block_table, cu_seqlens_q, kv_lens, q_pos0, int(max_q_len),
                            bool(causal), float(scale), float(softcap), lse)
        return (out, lse) if return_lse else out
    return attention_reference(q, k_cache, v_cache, block_table, cu_seqlens_q, kv_lens, q_pos0, causal, scale, softcap,
                               return_lse)


def pick_kv_splits(batch: int, num_kv_heads: int, head_dim_chunks: int, max_kv_len: int, num_sms: int = 148) -> int:
    """Number of KV splits.  A CTA walks its 64-token blocks one after the other (about a microsecond each) and the
    merge of the partials grows with the number of splits (about a tenth of that per split), so a small problem takes
    about sqrt(8 x blocks) splits; a large batch is limited to what still fits one wave of the grid (three CTAs of
    the split-KV kernel are resident per SM; a second, partly filled wave costs more than the extra parallelism
    brings).  At most 64."""
    blocks = max(1, (max_kv_len + 63) // 64)
    ctas = max(1, batch * num_kv_heads * head_dim_chunks)
    one_wave = max(1, (3 * num_sms) // ctas)
    want = max(1, math.ceil(math.sqrt(8.0 * blocks)))
    return int(max(1, min(want, one_wave, blocks, 64)))


FUSED_COMBINE_MAX_SPLITS = 32   # up to here the last split CTA merges the partials itself; beyond, a combine launch


def decode_workspace(batch: int, num_q_heads: int, head_dim: int, splits: int, device) -> torch.Tensor:
    return torch.empty(batch * num_q_heads * splits * (head_dim + 1), dtype=torch.float32, device=device)


_COUNTERS = {}


def _decode_counters(device, n: int) -> torch.Tensor:
    """Zeroed arrival counters of the fused split-KV combine, one buffer per device (the kernel leaves them zero)."""
    key = (device.type, device.index)
    buf = _COUNTERS.get(key)
    if buf is None or buf.numel() < n:
        buf = torch.zeros(max(n, 4096), dtype=torch.int32, device=device)
        _COUNTERS[key] = buf
    return buf


def gqa_fwd_batch_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                         workspace: Optional[torch.Tensor], q_lens, kv_lens: torch.Tensor, block_table: torch.Tensor,
                         scale: Optional[float] = None, soft_cap: float = 0.0, output_split=None, output_combine=None,
                         kv_split: int = -1, return_lse: bool = False):
    """Decode attention, one query token per sequence.  ``q`` [B, Hq, D] -> [B, Hq, D] (and the LSE [B, Hq])."""
    B, Hq, D = q.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if _native.use_native(q, k_cache, v_cache) and q.dtype == torch.bfloat16 and D in (64, 128):
        lib = _native.load(True)
        Hkv = k_cache.shape[2]
        group = Hq // Hkv
        splits = kv_split if kv_split > 0 else pick_kv_splits(B, Hkv, (group + 15) // 16,
                                                                k_cache.shape[1] * block_table.shape[1])
        need = B * Hq * splits * (D + 1)
        if workspace is None or workspace.numel() < need:
            workspace = decode_workspace(B, Hq, D, splits, q.device)
        out = output_combine if output_combine is not None else torch.empty_like(q)
        lse = torch.empty((B, Hq), dtype=torch.float32, device=q.device) if return_lse else None
        # without the LSE the last split CTA of every (sequence, KV head) merges the partials: one launch
        counters = None if (return_lse or splits > FUSED_COMBINE_MAX_SPLITS) else \
            _decode_counters(q.device, B * Hkv * ((group + 15) // 16))
        lib.decode_attn(q.contiguous(), k_cache, v_cache, block_table, kv_lens, workspace, int(splits), float(scale),
                        float(soft_cap), out, lse, None, counters)
        return (out, lse) if return_lse else out
    cu = torch.arange(B + 1, dtype=torch.int32, device=q.device)
    res = attention_reference(q, k_cache, v_cache, block_table, cu, kv_lens, None, False, scale, soft_cap, return_lse)
    return res


gqa_fwd_batch_decode_intra_rank = gqa_fwd_batch_decode
gqa_fwd_batch_decode_persistent = gqa_fwd_batch_decode


def merge_attention_partials(outs: torch.Tensor, lses: torch.Tensor) -> torch.Tensor:
    """LSE merge of partial attentions: ``outs`` [W, B, Hq, D], ``lses`` [W, B, Hq] -> [B, Hq, D] (fp32 reference)."""
    mx = lses.max(dim=0, keepdim=True).values
    w = torch.exp(lses - mx)
    w = torch.nan_to_num(w, nan=0.0)
    tot = w.sum(dim=0)
    res = (w.unsqueeze(-1) * outs.float()).sum(dim=0) / tot.clamp_min(1e-30).unsqueeze(-1)
    return res

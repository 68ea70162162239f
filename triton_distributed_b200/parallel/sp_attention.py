"""Sequence-parallel (context-parallel) prefill attention: all-gather of K/V, causal attention with zig-zag balancing.

API of the reference: ``create_sp_ag_attention_context_intra_node`` / ``fused_sp_ag_attn_intra_node``
(python/triton_dist/kernels/nvidia/sp_ag_attention_intra_node.py:59, :432).  Every rank holds Q/K/V of its sequence
shard; with ``enable_zig_zag`` the shard of rank r is the pair of chunks ``r`` and ``2W-1-r`` of every sequence so that
causal work is balanced.  K/V are all-gathered into a symmetric buffer (NVLS / push all-gather of this package) and
the attention kernel reads them as a *paged* cache whose block table undoes the zig-zag permutation, so no data is
re-ordered; the two chunks of a rank are two entries of the var-len batch with their own position offsets.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import _native, ops
from ..ops.allgather import create_fast_allgather_context, fast_allgather
from ..ops.common import ref_all_gather
from ..runtime import Runtime, get_runtime


@dataclass
class SPAllGatherAttentionContextIntraNode:
    rt: Runtime
    max_tokens_per_rank: int
    num_kv_heads: int
    head_dim: int
    dtype: torch.dtype
    k_buf: Optional[torch.Tensor] = None   # heap [W, max_tokens_per_rank, Hkv, D]
    v_buf: Optional[torch.Tensor] = None
    ag_ctx: object = None

    def finalize(self):
        if self.k_buf is not None:
            self.rt.symm_free(self.k_buf)
            self.rt.symm_free(self.v_buf)
            self.k_buf = None
        if self.ag_ctx is not None:
            self.ag_ctx.finalize()


def create_sp_ag_attention_context_intra_node(batch_size: int, q_heads: int, kv_heads: int, max_seqlen_k: int, head_dim: int,
                                              input_dtype: torch.dtype = torch.bfloat16, output_dtype=None, rank=None,
                                              local_rank=None, world_size=None, local_world_size=None, device=None):
    rt = get_runtime()
    W = rt.world_size
    per_rank = batch_size * ((max_seqlen_k + W - 1) // W)
    ctx = SPAllGatherAttentionContextIntraNode(rt, per_rank, kv_heads, head_dim, input_dtype)
    if rt.is_cuda and W > 1:
        ctx.k_buf = rt.symm_tensor((W, per_rank, kv_heads, head_dim), input_dtype, zero=False)
        ctx.v_buf = rt.symm_tensor((W, per_rank, kv_heads, head_dim), input_dtype, zero=False)
        ctx.ag_ctx = create_fast_allgather_context()
        torch.cuda.synchronize()
        rt.host_barrier()
    return ctx


create_sp_ag_attention_context_inter_node = create_sp_ag_attention_context_intra_node


def _chunks_of_rank(rank: int, W: int, zig_zag: bool):
    return [rank, 2 * W - 1 - rank] if zig_zag else [rank]


def fused_sp_ag_attn_intra_node(ctx: SPAllGatherAttentionContextIntraNode, q_shard: torch.Tensor, k_shard: torch.Tensor,
                                v_shard: torch.Tensor, output: Optional[torch.Tensor], cu_seqlens_q: torch.Tensor,
                                cu_seqlens_k: torch.Tensor, max_seqlen_q: int, max_seqlen_k: int, rank: Optional[int] = None,
                                world_size: Optional[int] = None, is_causal: bool = True, enable_zig_zag: bool = True):
    """q/k/v_shard: [tokens_local, heads, D] packed over the batch; ``cu_seqlens_q`` gives the LOCAL token ranges per
    sequence, ``cu_seqlens_k`` the GLOBAL lengths (each sequence length divisible by ``W``, or ``2W`` with zig-zag;
    the sequences may differ in length)."""
    rt = ctx.rt
    W = rt.world_size if world_size is None else world_size
    rank = rt.rank if rank is None else rank
    B = cu_seqlens_q.numel() - 1
    cu_q = cu_seqlens_q.tolist()
    cu_k = cu_seqlens_k.tolist()
    n_chunks = 2 * W if enable_zig_zag else W
    mine = _chunks_of_rank(rank, W, enable_zig_zag)
    # --- all-gather K / V
    t_local = k_shard.shape[0]
    if W > 1 and _native.use_native(k_shard):
        ctx.k_buf[rank, :t_local].copy_(k_shard)
        ctx.v_buf[rank, :t_local].copy_(v_shard)
        fast_allgather(ctx.k_buf, ctx.ag_ctx)
        fast_allgather(ctx.v_buf, ctx.ag_ctx)
        k_all, v_all = ctx.k_buf, ctx.v_buf                     # [W, per_rank, Hkv, D]
        per_rank = ctx.max_tokens_per_rank
    elif W > 1:
        k_all = ref_all_gather(k_shard.unsqueeze(0), rt.group)
        v_all = ref_all_gather(v_shard.unsqueeze(0), rt.group)
        per_rank = t_local
    else:
        k_all, v_all, per_rank = k_shard.unsqueeze(0), v_shard.unsqueeze(0), t_local
    Hkv, D = k_shard.shape[1], k_shard.shape[2]
    # --- paged view of the gathered K / V.  A rank holds, packed over the batch, its chunks of every sequence (chunk r,
    # and with zig-zag chunk 2W-1-r right behind it).  Sequences may differ in length: the page size is the largest
    # token count that divides every chunk length (and the per-rank stride of the gathered buffer), so that every chunk
    # is a whole number of pages and the block table can undo the zig-zag permutation without moving data.
    import math
    lens = [cu_k[b + 1] - cu_k[b] for b in range(B)]
    if any(l % n_chunks for l in lens) or any(l <= 0 for l in lens):
        raise ValueError("sp attention: every sequence length must be a positive multiple of the number of chunks "
                         f"({n_chunks})")
    chunk_of = [l // n_chunks for l in lens]
    cpr = len(mine)   # chunks per rank per sequence
    if sum(cpr * c for c in chunk_of) != t_local:
        raise ValueError("sp attention: the local shard does not hold cu_seqlens_k / world tokens of every sequence")
    page = math.gcd(*chunk_of, per_rank) if W > 1 else math.gcd(*chunk_of)
    k_pages = k_all.reshape(-1, Hkv, D)[: (W * per_rank) // page * page].reshape(-1, page, Hkv, D)
    v_pages = v_all.reshape(-1, Hkv, D)[: (W * per_rank) // page * page].reshape(-1, page, Hkv, D)
    pages_per_rank = per_rank // page
    # first local token of sequence b on any rank
    seq_off = [0]
    for c in chunk_of:
        seq_off.append(seq_off[-1] + cpr * c)
    dev = q_shard.device
    max_pages = max(lens) // page
    bt = torch.zeros((B, max_pages), dtype=torch.int32)
    for b in range(B):
        cb = chunk_of[b]
        ppc = cb // page                      # pages per chunk
        for c in range(n_chunks):
            if enable_zig_zag:
                owner, idx = (c, 0) if c < W else (2 * W - 1 - c, 1)
            else:
                owner, idx = c, 0
            first = owner * pages_per_rank + (seq_off[b] + idx * cb) // page
            bt[b, c * ppc:(c + 1) * ppc] = torch.arange(first, first + ppc, dtype=torch.int32)
    # --- var-len batch with one entry per (sequence, local chunk)
    entries_q, pos0, kv_len, table_rows = [0], [], [], []
    for b in range(B):
        for i, c in enumerate(mine):
            entries_q.append(entries_q[-1] + chunk_of[b])
            pos0.append(c * chunk_of[b])
            kv_len.append((c + 1) * chunk_of[b] if is_causal else lens[b])
            table_rows.append(b)
    max_q = max(chunk_of)
    cu = torch.tensor(entries_q, dtype=torch.int32, device=dev)
    q_pos0 = torch.tensor(pos0, dtype=torch.int32, device=dev)
    kv_lens = torch.tensor(kv_len, dtype=torch.int32, device=dev)
    table = bt[table_rows].contiguous().to(dev)
    out = ops.flash_attn_varlen(q_shard.contiguous(), k_pages.contiguous() if not k_pages.is_contiguous() else k_pages,
                                v_pages.contiguous() if not v_pages.is_contiguous() else v_pages, table, cu, kv_lens, max_q,
                                q_pos0=q_pos0, causal=is_causal, max_kv_len=max(kv_len))
    if output is not None:
        output.copy_(out)
        return output
    return out


fused_sp_ag_attn_inter_node = fused_sp_ag_attn_intra_node

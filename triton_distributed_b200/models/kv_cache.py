"""KV caches: dense per-sequence (``KV_Cache``, as python/triton_dist/models/kv_cache.py:29-66) and paged
(``PagedKVCache``, as mega_triton_kernel/models/paged_kv_cache.py:28-58).  Both expose the paged view the attention
kernels take: ``layer(i) -> (k, v) [pages, page_size, Hkv, D]`` plus an int32 ``block_table [B, max_pages]``.
Offsets live on the device so a CUDA graph of one decode step can be replayed while they advance."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..ops.attention import decode_workspace, pick_kv_splits


class KV_Cache:
    def __init__(self, num_layers: int, batch_size: int, max_length: int, kv_heads: int, head_dim: int,
                 dtype: torch.dtype = torch.bfloat16, device=None, world_size: int = 1):
        self.num_layers, self.batch_size, self.max_length = num_layers, batch_size, max_length
        self.kv_heads, self.head_dim = kv_heads, head_dim
        dev = device or "cuda"
        self.k_cache = torch.zeros(num_layers, batch_size, max_length, kv_heads, head_dim, dtype=dtype, device=dev)
        self.v_cache = torch.zeros_like(self.k_cache)
        self.kv_offset = torch.zeros(batch_size, dtype=torch.int32, device=dev)
        self.block_table = torch.arange(batch_size, dtype=torch.int32, device=dev).unsqueeze(1).contiguous()
        self._row_base = (torch.arange(batch_size, dtype=torch.int64, device=dev) * max_length)
        self._ws = None
        self.kv_splits = pick_kv_splits(batch_size, kv_heads, 1, max_length)

    # -- views used by the attention layer --------------------------------------------------------------------
    def layer(self, i: int) -> Tuple[torch.Tensor, torch.Tensor]:
        return self.k_cache[i], self.v_cache[i]

    def slots_for(self, position_ids: torch.Tensor, bsz: int, q_len: int) -> torch.Tensor:
        """Flat cache row of every token: ``b * max_length + position``."""
        return (self._row_base[:bsz, None] + position_ids.reshape(bsz, q_len).to(torch.int64)).reshape(-1)

    def kv_lens_after(self, q_len: int, bsz: int) -> torch.Tensor:
        return (self.kv_offset[:bsz] + q_len).to(torch.int32)

    def cu_seqlens(self, bsz: int, q_len: int) -> torch.Tensor:
        return torch.arange(0, (bsz + 1) * q_len, q_len, dtype=torch.int32, device=self.kv_offset.device)

    def decode_workspace(self, num_q_heads: int, head_dim: int) -> torch.Tensor:
        need = self.batch_size * num_q_heads * self.kv_splits * (head_dim + 1)
        if self._ws is None or self._ws.numel() < need:
            self._ws = decode_workspace(self.batch_size, num_q_heads, head_dim, self.kv_splits, self.kv_offset.device)
        return self._ws

    # -- per-step values shared by all layers (computed once instead of once per layer) ----------------------
    def begin_step(self, position_ids: torch.Tensor, bsz: int, q_len: int):
        self._step = (self.slots_for(position_ids, bsz, q_len), self.kv_lens_after(q_len, bsz), bsz, q_len)

    def end_step(self):
        self._step = None

    def step_values(self, position_ids: torch.Tensor, bsz: int, q_len: int):
        """(cache rows of the new tokens, kv lengths after the step): the values of ``begin_step`` when a step is
        open for the same shape, else computed here."""
        st = getattr(self, "_step", None)
        if st is not None and st[2] == bsz and st[3] == q_len:
            return st[0], st[1]
        return self.slots_for(position_ids, bsz, q_len), self.kv_lens_after(q_len, bsz)

    # -- bookkeeping ------------------------------------------------------------------------------------------
    def inc_offset(self, n: int = 1):
        self.kv_offset += n

    def clear(self):
        self.kv_offset.zero_()

    def rand_fill(self, length: int):
        """Pretend ``length`` tokens are cached (random contents): used by decode benchmarks."""
        self.k_cache[:, :, :length].normal_()
        self.v_cache[:, :, :length].normal_()
        self.kv_offset.fill_(length)


class PagedKVCache:
    """Pages of ``page_size`` tokens with a (random by default) block table, same interface as ``KV_Cache``."""

    def __init__(self, num_layers: int, batch_size: int, max_length: int, kv_heads: int, head_dim: int,
                 page_size: int = 16, dtype: torch.dtype = torch.bfloat16, device=None, shuffle: bool = True):
        dev = device or "cuda"
        self.num_layers, self.batch_size, self.max_length = num_layers, batch_size, max_length
        self.kv_heads, self.head_dim, self.page_size = kv_heads, head_dim, page_size
        self.pages_per_seq = (max_length + page_size - 1) // page_size
        n_pages = batch_size * self.pages_per_seq
        self.k_cache = torch.zeros(num_layers, n_pages, page_size, kv_heads, head_dim, dtype=dtype, device=dev)
        self.v_cache = torch.zeros_like(self.k_cache)
        order = torch.randperm(n_pages, device=dev) if shuffle else torch.arange(n_pages, device=dev)
        self.block_table = order.to(torch.int32).reshape(batch_size, self.pages_per_seq).contiguous()
        self.kv_offset = torch.zeros(batch_size, dtype=torch.int32, device=dev)
        self._ws = None
        self.kv_splits = pick_kv_splits(batch_size, kv_heads, 1, max_length)

    def layer(self, i: int):
        return self.k_cache[i], self.v_cache[i]

    def slots_for(self, position_ids: torch.Tensor, bsz: int, q_len: int) -> torch.Tensor:
        pos = position_ids.reshape(bsz, q_len).to(torch.int64)
        page = torch.gather(self.block_table[:bsz].to(torch.int64), 1, pos // self.page_size)
        return (page * self.page_size + pos % self.page_size).reshape(-1)

    kv_lens_after = KV_Cache.kv_lens_after
    cu_seqlens = KV_Cache.cu_seqlens
    decode_workspace = KV_Cache.decode_workspace
    inc_offset = KV_Cache.inc_offset
    clear = KV_Cache.clear
    begin_step = KV_Cache.begin_step
    end_step = KV_Cache.end_step
    step_values = KV_Cache.step_values

    def rand_fill(self, length: int):
        self.k_cache.normal_()
        self.v_cache.normal_()
        self.kv_offset.fill_(length)

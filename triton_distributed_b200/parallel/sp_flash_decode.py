"""Distributed flash-decode layer: KV sharded over ranks, one query token per sequence.

API of the reference: ``SpGQAFlashDecodeAttention`` (python/triton_dist/layers/nvidia/sp_flash_decode_layer.py:44-185).
Each rank runs split-KV attention over its KV shard.  While the head chunks (batch x KV heads x ceil(group / 16)) fit
the SMs the whole step is ONE launch (``csrc/attn.cu`` ``decode_splitkv_dist_kernel``): the last split CTA of a head
chunk merges the local splits, pushes (out, LSE) to every rank as 8-byte packets with the call epoch in band, waits for
the W packets of its heads and merges them by LSE.  Larger problems use split-KV plus one exchange-and-merge launch
(``dist_combine_kernel``).  The reference runs split-KV, a combine, an LL all-gather and a second combine
(python/triton_dist/kernels/nvidia/flash_decode.py:587-760, sp_flash_decode_layer.py:120-185).
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import _native
from ..ops.attention import attention_reference, decode_workspace, merge_attention_partials, pick_kv_splits
from ..ops.common import new_ctx_dev, ref_all_gather
from ..runtime import get_runtime


ONE_LAUNCH_MAX_SPLITS = 16


class SpGQAFlashDecodeAttention:
    def __init__(self, rank: int, node: int, num_ranks: int, num_nodes: int, num_q_heads: int, num_kv_heads: int,
                 q_head_dim: int, v_head_dim: int, page_size: int = 1, scale: Optional[float] = None,
                 soft_cap: float = 0.0, max_allowed_batch: int = 1, thrink_buffer_threshold: int = 500,
                 stages: int = 20):
        self.rt = get_runtime()
        self.rank, self.num_ranks = rank, num_ranks
        self.num_q_heads, self.num_kv_heads = num_q_heads, num_kv_heads
        self.head_dim = q_head_dim
        assert q_head_dim == v_head_dim, "q and v head dims must match"
        self.page_size = page_size
        self.scale = scale if scale is not None else 1.0 / math.sqrt(q_head_dim)
        self.soft_cap = soft_cap
        self.max_batch = max_allowed_batch
        self.staging = None
        self.ctx_dev = None
        self.workspace = None
        self.counters = None
        # None: one launch while the local KV is cut into at most ONE_LAUNCH_MAX_SPLITS splits.  Beyond that the merge of
        # the splits by a single CTA per KV head costs more than the second launch saves (bs 1, 16 k KV per rank, 45
        # splits, two B200: 39 us in one launch, 34 us in two).  True / False force a form.
        self.one_launch: Optional[bool] = None
        self.last_launches = 0
        if self.rt.is_cuda and num_ranks > 1:
            packets = num_ranks * max_allowed_batch * num_q_heads * (q_head_dim + 1)
            self.staging = self.rt.symm_tensor((2, packets, 2), torch.int32)   # 8-byte packets
            self.ctx_dev = new_ctx_dev(self.rt)
            chunks = max_allowed_batch * num_kv_heads * ((num_q_heads // num_kv_heads + 15) // 16)
            self.counters = torch.zeros(chunks, dtype=torch.int32, device=self.rt.device)
            torch.cuda.synchronize()
            self.rt.host_barrier()

    def forward(self, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, global_kv_lens: torch.Tensor,
                block_table: torch.Tensor) -> torch.Tensor:
        """q [B, Hq, D] replicated; k/v cache: this rank's shard; global_kv_lens [W, B] int32."""
        B, Hq, D = q.shape
        local_lens = global_kv_lens[self.rank].contiguous()
        if not _native.use_native(q, k_cache, v_cache):
            cu = torch.arange(B + 1, dtype=torch.int32, device=q.device)
            out, lse = attention_reference(q, k_cache, v_cache, block_table, cu, local_lens, None, False, self.scale,
                                           self.soft_cap, True)
            if self.num_ranks == 1:
                return out
            outs = ref_all_gather(out.float().unsqueeze(0), self.rt.group)
            lses = ref_all_gather(lse.t().contiguous().unsqueeze(0), self.rt.group)
            return merge_attention_partials(outs, lses).to(q.dtype)
        lib = _native.load(True)
        if B > self.max_batch:
            raise ValueError(f"batch {B} exceeds max_allowed_batch {self.max_batch}")
        group = Hq // self.num_kv_heads
        splits = pick_kv_splits(B, self.num_kv_heads, (group + 15) // 16, k_cache.shape[1] * block_table.shape[1])
        need = B * Hq * splits * (D + 1)
        if self.workspace is None or self.workspace.numel() < need:
            self.workspace = decode_workspace(B, Hq, D, splits, q.device)
        out = torch.empty_like(q)
        if self.num_ranks == 1:
            lib.decode_attn(q.contiguous(), k_cache, v_cache, block_table, local_lens, self.workspace, splits,
                            float(self.scale), float(self.soft_cap), out, None, None, None)
            return out
        self.last_launches = lib.dist_decode_attn(
            self.rt.heap, q.contiguous(), k_cache, v_cache, block_table, local_lens, self.workspace, splits,
            float(self.scale), float(self.soft_cap), out, self.staging, self.ctx_dev, self.rt.config.wait_timeout_s,
            self.counters if (self.one_launch if self.one_launch is not None else splits <= ONE_LAUNCH_MAX_SPLITS) else None)
        return out

    __call__ = forward

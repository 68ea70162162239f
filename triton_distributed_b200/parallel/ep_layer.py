"""Expert-parallel MoE layers: the dispatch / combine transport (``EPAll2AllLayer``) and a full EP MoE block.

API of the reference: ``EPAll2AllLayer`` (python/triton_dist/layers/nvidia/ep_a2a_layer.py:50-341) with ``dispatch`` /
``combine``; the full block mirrors the reference's EP inference test (test/nvidia/test_ep_moe_inference.py:317-457):
router -> dispatch -> grouped GEMMs on the local experts -> combine.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..runtime import get_runtime


class EPAll2AllLayer:
    def __init__(self, ep_group=None, max_tokens: int = 128, hidden: int = 7168, topk: int = 8, rank: Optional[int] = None,
                 num_tot_experts: int = 256, local_world_size: Optional[int] = None, world_size: Optional[int] = None,
                 dtype: torch.dtype = torch.bfloat16, quant: bool = False, layout: str = "packed"):
        rt = get_runtime()
        self.rt = rt
        self.rank = rt.rank if rank is None else rank
        self.world_size = rt.world_size if world_size is None else world_size
        self.ctx = ops.create_all_to_all_context(max_tokens, hidden, self.rank, num_tot_experts, self.world_size,
                                                 num_tot_experts // self.world_size, dtype, topk=topk, quant=quant,
                                                 layout=layout)
        self._recv = None
        self._weights = None

    def dispatch(self, input: torch.Tensor, exp_indices: torch.Tensor, weight: Optional[torch.Tensor] = None):
        """input [T, H], exp_indices [T, k] -> (rows of the local experts sorted by expert and padded to 128,
        the sort describing them).  The routing weights are kept for ``combine``."""
        self._recv = ops.ep_dispatch(self.ctx, input, exp_indices)
        self._weights = weight
        return self._recv.x_sorted, self._recv.sort

    def combine(self, input: torch.Tensor) -> torch.Tensor:
        """input: expert outputs in the layout ``dispatch`` returned -> [T, H] (weighted sum over the k slots)."""
        return ops.ep_combine(self.ctx, input, self._recv, self._weights)

    def finalize(self):
        self.ctx.finalize()


class EP_MoE:
    """Experts sharded over ranks (E/W per rank, full intermediate size)."""

    def __init__(self, hidden: int, inter: int, num_experts: int, topk: int, max_tokens: int, quant: bool = True,
                 layout: str = "ll", dtype: torch.dtype = torch.bfloat16, seed: int = 0, norm_topk: bool = True):
        rt = get_runtime()
        self.rt, self.rank, self.world_size = rt, rt.rank, rt.world_size
        self.num_experts, self.topk, self.hidden, self.inter = num_experts, topk, hidden, inter
        self.epr = num_experts // self.world_size
        self.norm_topk = norm_topk
        g = torch.Generator(device=rt.device).manual_seed(seed)    # same stream on every rank: slice out the local experts
        router = (torch.randn(num_experts, hidden, device=rt.device, generator=g) * 0.02).to(dtype)
        self.router_w = router
        lo = self.rank * self.epr
        self.full_w13 = None
        self.w13 = torch.empty(self.epr, 2 * inter, hidden, device=rt.device, dtype=dtype)
        self.w2 = torch.empty(self.epr, hidden, inter, device=rt.device, dtype=dtype)
        for e in range(num_experts):
            a = (torch.randn(2 * inter, hidden, device=rt.device, generator=g) * 0.02).to(dtype)
            b = (torch.randn(hidden, inter, device=rt.device, generator=g) * 0.02).to(dtype)
            if lo <= e < lo + self.epr:
                self.w13[e - lo], self.w2[e - lo] = a, b
        self.a2a = EPAll2AllLayer(max_tokens=max_tokens, hidden=hidden, topk=topk, num_tot_experts=num_experts, dtype=dtype,
                                  quant=quant, layout=layout)

    def route(self, x: torch.Tensor):
        return ops.topk_router(ops.gemm(x, self.router_w).float(), self.topk, self.norm_topk)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        ids, w = self.route(x)
        xs, srt = self.a2a.dispatch(x, ids, w)
        h = ops.silu_mul(ops.group_gemm_sorted(xs, self.w13, srt))
        y = ops.group_gemm_sorted(h, self.w2, srt)
        return self.a2a.combine(y)

    __call__ = forward

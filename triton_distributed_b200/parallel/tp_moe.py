"""Tensor-parallel MoE block: experts replicated over the ranks, intermediate dimension sharded.

API of the reference: ``TP_MoE`` (python/triton_dist/layers/nvidia/tp_moe.py:48-279): router (softmax + top-k),
all-gather of the routing, AG -> grouped GEMM (gate/up), activation, grouped GEMM -> top-k reduce -> reduce-scatter
(or all-reduce).  Here the router is an own kernel, the routing is gathered with the packet all-gather instead of NCCL,
and the two grouped GEMMs stay in the expert-sorted layout (no scatter / re-gather between them).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .. import ops
from ..runtime import get_runtime


class TP_MoE:
    def __init__(self, rank: int = 0, world_size: int = 1, group=None):
        self.rank, self.world_size, self.group = rank, world_size, group
        self.router_w: Optional[torch.Tensor] = None   # [E, H]
        self.w13: Optional[torch.Tensor] = None        # [E, 2*I/W, H]  gate rows then up rows
        self.w2: Optional[torch.Tensor] = None         # [E, H, I/W]
        self.ag_ctx = self.rs_ctx = self.ll_ctx = None
        self.norm_topk = True

    def _init_parameters(self, router: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, topk: int,
                         norm_topk: bool = True, device=None):
        """router [E, H]; gate / up [E, I, H]; down [E, H, I] (full); shards the intermediate dimension."""
        device = device or get_runtime().device
        W, r = self.world_size, self.rank
        I = gate.shape[1]
        il = I // W
        self.router_w = router.to(device).contiguous()
        self.w13 = torch.cat([gate[:, r * il:(r + 1) * il], up[:, r * il:(r + 1) * il]], dim=1).to(device).contiguous()
        self.w2 = down[:, :, r * il:(r + 1) * il].to(device).contiguous()
        self.num_experts, self.topk, self.norm_topk = router.shape[0], topk, norm_topk
        self.hidden, self.inter_local = router.shape[1], il

    def init_random(self, hidden: int, inter: int, num_experts: int, topk: int, dtype=torch.bfloat16, device=None,
                    std: float = 0.02, seed: int = 0):
        device = device or get_runtime().device
        g = torch.Generator(device=device).manual_seed(seed)          # router: replicated
        self.router_w = (torch.randn(num_experts, hidden, device=device, generator=g) * std).to(dtype)
        g2 = torch.Generator(device=device).manual_seed(seed + 15485863 * (self.rank + 1))
        il = inter // self.world_size
        self.w13 = (torch.randn(num_experts, 2 * il, hidden, device=device, generator=g2) * std).to(dtype)
        self.w2 = (torch.randn(num_experts, hidden, il, device=device, generator=g2) * std).to(dtype)
        self.num_experts, self.topk = num_experts, topk
        self.hidden, self.inter_local = hidden, il

    def _init_ctx(self, max_M: int, **kw):
        self.ag_ctx = ops.create_ag_group_gemm_context(max_M, 2 * self.inter_local, self.hidden, self.num_experts, self.topk,
                                                       dtype=self.w13.dtype)
        self.rs_ctx = ops.create_moe_rs_context(max_token_num=max_M, hidden_dim=self.hidden, num_experts=self.num_experts,
                                                topk=self.topk, input_dtype=self.w13.dtype)
        if self.world_size > 1 and get_runtime().is_cuda:
            self.ll_ctx = ops.create_fast_allgather_context(max_ll_bytes=max(64 * 1024, max_M * self.topk * 8))

    def finalize(self):
        for c in (self.ag_ctx, self.rs_ctx, self.ll_ctx):
            if c is not None:
                c.finalize()
        self.ag_ctx = self.rs_ctx = self.ll_ctx = None

    def _route(self, x: torch.Tensor):
        logits = ops.gemm(x, self.router_w).float()
        return ops.topk_router(logits, self.topk, self.norm_topk)

    def torch_fwd(self, x: torch.Tensor) -> torch.Tensor:
        """Golden path.  x [T, H] replicated -> [T, H] replicated (partial sums all-reduced with NCCL / gloo)."""
        ids, w = ops.topk_router_reference(torch.matmul(x, self.router_w.t()).float(), self.topk, self.norm_topk)
        h = ops.group_gemm_reference(x, self.w13, ids)
        h = ops.elementwise.silu_mul_reference(h)
        o = ops.moe_reduce_reference(h, self.w2, ids, w)
        if self.world_size > 1:
            dist.all_reduce(o, group=self.group)
        return o

    def dist_triton_fwd(self, x: torch.Tensor) -> torch.Tensor:
        """x [T/W, H] (row shard) -> [T/W, H]: route locally, gather routing, AG+grouped GEMM, act, grouped GEMM+RS."""
        ids, w = self._route(x)
        if self.world_size > 1:
            if x.is_cuda and self.ll_ctx is not None and ids.numel() * 4 <= self.ll_ctx.max_ll_bytes and (ids.numel() * 4) % 8 == 0:
                ids = ops.all_gather_ll(ids, self.ll_ctx).reshape(-1, self.topk)
                w = ops.all_gather_ll(w, self.ll_ctx).reshape(-1, self.topk)
            else:
                ids = ops.all_gather(ids)
                w = ops.all_gather(w)
        hs, srt = ops.ag_group_gemm(x, self.w13, self.ag_ctx, ids, sorted_output=True)
        act = ops.silu_mul(hs)
        return ops.run_moe_reduce_rs(act, self.w2, ids, w, self.rs_ctx, sort=srt)

    def dist_triton_AR_fwd(self, x: torch.Tensor) -> torch.Tensor:
        """x [T, H] replicated -> [T, H] replicated (grouped GEMMs + all-reduce)."""
        ids, w = self._route(x)
        srt = ops.sort_topk_ids_align_block_size(ids, self.num_experts)
        hs = ops.group_gemm_gather(x, self.w13, srt, a_row_div=self.topk)   # token rows gathered inside the GEMM
        act = ops.silu_mul(hs)
        return ops.run_moe_reduce_ar(act, self.w2, ids, w, self.rs_ctx, sort=srt)

    def set_fwd(self, mode: str = "torch"):
        self.fwd = {"torch": self.torch_fwd, "triton_dist": self.dist_triton_fwd, "ag_rs": self.dist_triton_fwd,
                    "triton_dist_AR": self.dist_triton_AR_fwd, "allreduce": self.dist_triton_AR_fwd,
                    "triton_dist_gemm_ar": self.dist_triton_AR_fwd, "gemm_ar": self.dist_triton_AR_fwd}[mode]

    def __call__(self, x):
        return self.fwd(x)

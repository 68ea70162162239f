"""Tensor-parallel SwiGLU MLP with four communication modes.

API of the reference: ``TP_MLP`` (python/triton_dist/layers/nvidia/tp_mlp.py:52-274): ``_init_parameters`` shards
and fuses gate/up (column parallel) and down (row parallel); ``torch_fwd`` is the NCCL + cuBLAS golden path;
``dist_triton_fwd`` = AG-GEMM -> act -> GEMM-RS on row-sharded activations; ``dist_triton_AR_fwd`` = GEMMs + the
all-reduce library; ``dist_triton_gemm_ar_fwd`` = GEMM + fused GEMM-AllReduce.  The method names are kept so code
written against the reference runs unchanged; here they dispatch to the sm_100a kernels of this package.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .. import ops
from ..runtime import get_runtime


def shard_rows(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = w.shape[0] // world
    return w[rank * n:(rank + 1) * n]


def shard_cols(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = w.shape[1] // world
    return w[:, rank * n:(rank + 1) * n]


class TP_MLP:
    def __init__(self, rank: int = 0, world_size: int = 1, group=None):
        self.rank, self.world_size, self.group = rank, world_size, group
        self.gate_up_proj: Optional[torch.Tensor] = None   # [2*I/W, H]: gate rows then up rows of this rank
        self.down_proj: Optional[torch.Tensor] = None      # [H, I/W]
        self.ag_ctx = self.rs_ctx = self.ar_ctx = self.gemm_ar_ctx = None
        self.act_fn = "silu"

    # -- parameters -----------------------------------------------------------------------------------------
    def _init_parameters(self, mlp=None, gate: Optional[torch.Tensor] = None, up: Optional[torch.Tensor] = None,
                         down: Optional[torch.Tensor] = None, device=None, verbose: bool = False):
        """Shard full weights: gate/up [I, H] by rows (column parallel), down [H, I] by columns (row parallel).
        ``mlp`` may be an HF module with ``gate_proj`` / ``up_proj`` / ``down_proj`` Linear layers."""
        if mlp is not None:
            gate, up, down = mlp.gate_proj.weight.detach(), mlp.up_proj.weight.detach(), mlp.down_proj.weight.detach()
        device = device or get_runtime().device
        g = shard_rows(gate, self.rank, self.world_size)
        u = shard_rows(up, self.rank, self.world_size)
        self.gate_up_proj = torch.cat([g, u], dim=0).to(device).contiguous()
        self.down_proj = shard_cols(down, self.rank, self.world_size).to(device).contiguous()
        self.hidden, self.inter_local = self.down_proj.shape[0], self.down_proj.shape[1]

    def init_random(self, hidden: int, intermediate: int, dtype=torch.bfloat16, device=None, std: float = 0.02, seed: int = 0):
        device = device or get_runtime().device
        g = torch.Generator(device=device).manual_seed(seed + 7919 * self.rank)
        il = intermediate // self.world_size
        self.gate_up_proj = (torch.randn(2 * il, hidden, device=device, generator=g) * std).to(dtype)
        self.down_proj = (torch.randn(hidden, il, device=device, generator=g) * std).to(dtype)
        self.hidden, self.inter_local = hidden, il

    # -- contexts -------------------------------------------------------------------------------------------
    def _init_ctx(self, max_M: int, **kw):
        self.ag_ctx = ops.create_ag_gemm_context(max_M=max_M, K=self.hidden, dtype=self.gate_up_proj.dtype)
        self.rs_ctx = ops.create_gemm_rs_context(max_M=max_M, N=self.hidden, output_dtype=self.gate_up_proj.dtype)

    def _init_AR_ctx(self, max_M: int, **kw):
        self.ar_ctx = ops.create_allreduce_ctx(max(4 * max_M * self.hidden * 2, 1 << 20))

    def _init_gemm_ar_ctx(self, max_M: int, **kw):
        self.gemm_ar_ctx = ops.create_gemm_ar_context(max_M=max_M, N=self.hidden, dtype=self.gate_up_proj.dtype)

    def finalize(self):
        for c in (self.ag_ctx, self.rs_ctx, self.ar_ctx, self.gemm_ar_ctx):
            if c is not None:
                c.finalize()
        self.ag_ctx = self.rs_ctx = self.ar_ctx = self.gemm_ar_ctx = None

    # -- forwards -------------------------------------------------------------------------------------------
    def torch_fwd(self, x: torch.Tensor) -> torch.Tensor:
        """Golden path: cuBLAS GEMMs + NCCL all-reduce; x [M, H] replicated -> [M, H] replicated."""
        h = torch.matmul(x, self.gate_up_proj.t())
        i = h.shape[-1] // 2
        h = torch.nn.functional.silu(h[..., :i]) * h[..., i:]
        o = torch.matmul(h, self.down_proj.t())
        if self.world_size > 1:
            dist.all_reduce(o, group=self.group)
        return o

    def dist_triton_fwd(self, x: torch.Tensor) -> torch.Tensor:
        """AG-GEMM -> SiLU*up -> GEMM-RS.  x [M/W, H] (row shard) -> [M/W, H] (row shard)."""
        h = ops.ag_gemm(x, self.gate_up_proj, self.ag_ctx)
        h = ops.silu_mul(h)
        return ops.gemm_rs(h, self.down_proj, self.rs_ctx)

    def dist_triton_AR_fwd(self, x: torch.Tensor) -> torch.Tensor:
        """Own GEMMs + the all-reduce library; x replicated."""
        h = ops.silu_mul(ops.gemm(x, self.gate_up_proj))
        o = ops.gemm(h, self.down_proj)
        return ops.all_reduce(o, ctx=self.ar_ctx) if self.world_size > 1 else o

    def dist_triton_gemm_ar_fwd(self, x: torch.Tensor) -> torch.Tensor:
        """GEMM -> act -> fused GEMM+AllReduce (decode sizes); x replicated."""
        h = ops.silu_mul(ops.gemm(x, self.gate_up_proj))
        return ops.gemm_allreduce_op(self.gemm_ar_ctx, h, self.down_proj)

    # per-op entry points used by the layer benchmarks of the reference (tp_mlp.py:231-274)
    def torch_ag_gemm(self, x):
        return ops.ag_gemm_reference(x, self.gate_up_proj, self.group)

    def dist_triton_ag_gemm(self, x):
        return ops.ag_gemm(x, self.gate_up_proj, self.ag_ctx)

    def torch_gemm_rs(self, x):
        return ops.gemm_rs_reference(x, self.down_proj, self.group)

    def dist_triton_gemm_rs(self, x):
        return ops.gemm_rs(x, self.down_proj, self.rs_ctx)

    def set_fwd(self, mode: str = "torch"):
        self.fwd = {"torch": self.torch_fwd, "triton_dist": self.dist_triton_fwd, "ag_rs": self.dist_triton_fwd,
                    "triton_dist_AR": self.dist_triton_AR_fwd, "allreduce": self.dist_triton_AR_fwd,
                    "triton_dist_gemm_ar": self.dist_triton_gemm_ar_fwd, "gemm_ar": self.dist_triton_gemm_ar_fwd}[mode]

    def __call__(self, x):
        return self.fwd(x)

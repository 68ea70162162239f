"""Tensor-parallel mixture-of-experts ops: router, token sort, grouped GEMM, AG -> grouped GEMM, grouped GEMM -> top-k
reduce -> reduce-scatter / all-reduce.

API of the reference: ``create_ag_group_gemm_context`` / ``ag_group_gemm`` (kernels/nvidia/allgather_group_gemm.py:337, :401),
``create_moe_rs_context`` / ``run_moe_reduce_rs`` (moe_reduce_rs.py:87, :710), ``run_moe_reduce_ar`` (moe_reduce_ar.py:482),
index helpers of moe_utils.py.  Expert weights are stored ``[E, N, K]`` (K-major rows, the layout the tcgen05 kernel
loads with TMA); the reference's ``[E, K, N]`` tensors are ``w.transpose(1, 2).contiguous()`` of these.

GPU path: ``csrc/moe.cu`` (router / sort / gather / reduce) + the grouped mode of ``csrc/gemm_sm100.cu``; tokens are
all-gathered with the NVLS / push all-gather of this package and the final cross-rank sum uses its reduce-scatter /
all-reduce kernels.  CPU path and oracle: the torch restatements below.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from .. import _native
from ..runtime import Runtime, get_runtime
from .allgather import create_fast_allgather_context, fast_allgather
from .allreduce import all_reduce, create_allreduce_ctx
from .common import ref_all_gather, ref_all_reduce, ref_reduce_scatter
from .reduce_scatter import create_reduce_scater_2d_ctx, reduce_scatter_2d_op

BLOCK_M = 128


# ------------------------------------------------------------------ torch references
def topk_router_reference(logits: torch.Tensor, k: int, normalize: bool = True):
    p = torch.softmax(logits.float(), dim=-1)
    w, ids = torch.topk(p, k, dim=-1)
    if normalize:
        w = w / w.sum(-1, keepdim=True)
    return ids.to(torch.int32), w


def group_gemm_reference(x: torch.Tensor, w: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
    """x [T, K], w [E, N, K], topk_ids [T, k] -> y [T*k, N] in (token, slot) order (fp32 math)."""
    T, k = topk_ids.shape
    out = torch.zeros(T * k, w.shape[1], dtype=torch.float32, device=x.device)
    flat = topk_ids.reshape(-1).long()
    xx = x.float().repeat_interleave(k, dim=0)
    for e in range(w.shape[0]):
        sel = (flat == e).nonzero(as_tuple=True)[0]
        if sel.numel():
            out[sel] = xx[sel] @ w[e].float().t()
    return out.to(x.dtype)


def moe_reduce_reference(y: torch.Tensor, w2: torch.Tensor, topk_ids: torch.Tensor, topk_w: torch.Tensor) -> torch.Tensor:
    """y [T*k, K2] (token, slot order), w2 [E, H, K2] -> [T, H] = sum_j weight * (y_j @ w2[e_j]^T)."""
    T, k = topk_ids.shape
    flat = topk_ids.reshape(-1).long()
    out = torch.zeros(T * k, w2.shape[1], dtype=torch.float32, device=y.device)
    for e in range(w2.shape[0]):
        sel = (flat == e).nonzero(as_tuple=True)[0]
        if sel.numel():
            out[sel] = y[sel].float() @ w2[e].float().t()
    out = out.reshape(T, k, -1) * topk_w.float().unsqueeze(-1)
    return out.sum(1).to(y.dtype)


# ------------------------------------------------------------------ single-GPU building blocks
def topk_router(logits: torch.Tensor, k: int, normalize: bool = True):
    """softmax + top-k: int32 ids [T, k], fp32 weights [T, k]."""
    if _native.use_native(logits) and logits.shape[-1] <= 512 and k <= 32:
        ids, w = _native.load(True).topk_router(logits.float().contiguous(), int(k), bool(normalize))
        return ids, w
    return topk_router_reference(logits, k, normalize)


@dataclass
class MoESort:
    sorted_ids: torch.Tensor    # [cap] flat (token*k+slot) per sorted row, -1 = padding
    pos_of: torch.Tensor        # [T*k] sorted row of every pair
    tile_expert: torch.Tensor   # [cap/128]
    offsets: torch.Tensor       # [E+1] padded start row of every expert
    meta: torch.Tensor          # [padded rows, tiles]
    counts: torch.Tensor        # [E]
    k: int


def sort_topk_ids_align_block_size(topk_ids: torch.Tensor, num_experts: int, block_size: int = BLOCK_M) -> MoESort:
    """Sort (token, slot) pairs by expert, every expert padded to a multiple of ``block_size`` rows."""
    k = topk_ids.shape[-1]
    if _native.use_native(topk_ids):
        s, p, t, o, m, c = _native.load(True).moe_align_sort(topk_ids.to(torch.int32).contiguous(), int(num_experts),
                                                             int(block_size))
        return MoESort(s, p, t, o, m, c, k)
    flat = topk_ids.reshape(-1).long()
    n = flat.numel()
    counts = torch.bincount(flat[(flat >= 0) & (flat < num_experts)], minlength=num_experts)
    padded = (counts + block_size - 1) // block_size * block_size
    offsets = torch.zeros(num_experts + 1, dtype=torch.long)
    offsets[1:] = padded.cumsum(0)
    cap = n + num_experts * (block_size - 1)
    cap = max(block_size, (cap + block_size - 1) // block_size * block_size)
    sorted_ids = torch.full((cap,), -1, dtype=torch.int32)
    pos_of = torch.full((max(n, 1),), -1, dtype=torch.int32)
    cursor = offsets[:-1].clone()
    for i in range(n):
        e = int(flat[i])
        if 0 <= e < num_experts:
            sorted_ids[cursor[e]] = i
            pos_of[i] = cursor[e]
            cursor[e] += 1
    tile_expert = torch.full((cap // block_size,), -1, dtype=torch.int32)
    for e in range(num_experts):
        tile_expert[offsets[e] // block_size:offsets[e + 1] // block_size] = e
    meta = torch.tensor([int(offsets[-1]), int(offsets[-1]) // block_size], dtype=torch.int32)
    return MoESort(sorted_ids, pos_of, tile_expert, offsets.to(torch.int32), meta, counts.to(torch.int32), k)


calc_gather_scatter_index = sort_topk_ids_align_block_size


def tile_arrival_order(srt: MoESort, tokens_per_rank: int, rank: int, world: int, block_size: int = BLOCK_M):
    """Visiting order of the ``block_size``-row tiles of an expert-sorted layout while the token shards of a ring
    all-gather arrive: ``(order, stage)`` with ``stage[t]`` the largest ring distance of the source ranks of tile
    ``t``'s rows (-1: padding only) and ``order`` the tiles by stage, expert order kept inside a stage.  Computed on the
    host by the C++ reference (``csrc/moe_sched.cc``) when the native library is there, else in Python; the reference's
    ``threadblock_swizzle_ag_moe`` kernels produce the same order (threadblock_swizzle_ag_moe_triton.py:96-216)."""
    lib = _native.load(False)
    if lib is not None:
        o, st = lib.moe_tile_arrival_order(srt.sorted_ids, int(srt.k), int(tokens_per_rank), int(rank), int(world),
                                           int(block_size))
        return o, st
    ids = srt.sorted_ids.cpu().tolist()
    tiles = (len(ids) + block_size - 1) // block_size
    stage = []
    for t in range(tiles):
        s = -1
        for i in ids[t * block_size:(t + 1) * block_size]:
            if i >= 0:
                s = max(s, ((i // srt.k) // tokens_per_rank - rank) % world)
        stage.append(s)
    order = sorted(range(tiles), key=lambda t: world if stage[t] < 0 else stage[t])
    return torch.tensor(order, dtype=torch.int32), torch.tensor(stage, dtype=torch.int32)


def group_gemm_sorted(a_sorted: torch.Tensor, w: torch.Tensor, srt: MoESort) -> torch.Tensor:
    """Rows sorted by expert [cap, K] x w [E, N, K] -> [cap, N] (rows of skipped tiles are left unwritten)."""
    if _native.use_native(a_sorted, w) and a_sorted.dtype == torch.bfloat16:
        out = torch.empty((a_sorted.shape[0], w.shape[1]), dtype=a_sorted.dtype, device=a_sorted.device)
        _native.load(True).group_gemm_bf16(a_sorted, w.contiguous(), out, srt.tile_expert, 0, 0)
        return out
    out = torch.zeros((a_sorted.shape[0], w.shape[1]), dtype=a_sorted.dtype, device=a_sorted.device)
    te = srt.tile_expert.tolist()
    for t, e in enumerate(te):
        if e >= 0:
            out[t * BLOCK_M:(t + 1) * BLOCK_M] = (a_sorted[t * BLOCK_M:(t + 1) * BLOCK_M].float() @ w[e].float().t()).to(out.dtype)
    return out


def gather_sorted(x: torch.Tensor, srt: MoESort) -> torch.Tensor:
    if _native.use_native(x) and x.dtype == torch.bfloat16:
        return _native.load(True).moe_gather(x, srt.sorted_ids, srt.meta, int(srt.k))
    ids = srt.sorted_ids.long()
    out = torch.zeros((ids.numel(), x.shape[1]), dtype=x.dtype, device=x.device)
    ok = ids >= 0
    out[ok] = x[ids[ok] // srt.k]
    return out


def reduce_topk(y_sorted: torch.Tensor, srt: MoESort, topk_w: Optional[torch.Tensor], num_tokens: int) -> torch.Tensor:
    """[T, H] = sum over the k slots of weight * sorted row."""
    if _native.use_native(y_sorted) and y_sorted.dtype == torch.bfloat16:
        w = topk_w.float().contiguous() if topk_w is not None else None
        return _native.load(True).moe_topk_reduce(y_sorted.contiguous(), srt.pos_of, w, int(num_tokens), int(srt.k))
    pos = srt.pos_of[:num_tokens * srt.k].long().reshape(num_tokens, srt.k)
    rows = y_sorted.float()[pos.clamp_min(0)]
    rows = rows * (pos >= 0).unsqueeze(-1)
    if topk_w is not None:
        rows = rows * topk_w.float().unsqueeze(-1)
    return rows.sum(1).to(y_sorted.dtype)


def unsort(y_sorted: torch.Tensor, srt: MoESort, rows: int) -> torch.Tensor:
    if _native.use_native(y_sorted) and y_sorted.dtype == torch.bfloat16:
        return _native.load(True).moe_unsort(y_sorted.contiguous(), srt.pos_of, int(rows))
    pos = srt.pos_of[:rows].long()
    out = y_sorted[pos.clamp_min(0)].clone()
    out[pos < 0] = 0
    return out


# ------------------------------------------------------------------ AG -> grouped GEMM
@dataclass
class MoEAgScatterGroupGemmContext:
    rt: Runtime
    rank: int
    num_ranks: int
    max_ntokens: int
    N_per_rank: int
    K: int
    num_experts: int
    topk: int
    dtype: torch.dtype
    ag_buffer: Optional[torch.Tensor] = None    # heap [max_ntokens, K]
    ag_ctx: object = None
    last_sort: Optional[MoESort] = None

    def finalize(self):
        if self.ag_buffer is not None:
            self.rt.symm_free(self.ag_buffer)
            self.ag_buffer = None
        if self.ag_ctx is not None:
            self.ag_ctx.finalize()
            self.ag_ctx = None


def create_ag_group_gemm_context(max_ntokens: int, N_per_rank: int, K: int, num_experts: int, topk: int,
                                 dtype: torch.dtype = torch.bfloat16, rank: Optional[int] = None,
                                 num_ranks: Optional[int] = None, **kw) -> MoEAgScatterGroupGemmContext:
    rt = get_runtime()
    rank = rt.rank if rank is None else rank
    num_ranks = rt.world_size if num_ranks is None else num_ranks
    ctx = MoEAgScatterGroupGemmContext(rt, rank, num_ranks, max_ntokens, N_per_rank, K, num_experts, topk, dtype)
    if rt.is_cuda and num_ranks > 1:
        ctx.ag_buffer = rt.symm_tensor((max_ntokens, K), dtype, zero=False)
        ctx.ag_ctx = create_fast_allgather_context()
        torch.cuda.synchronize()
        rt.host_barrier()
    return ctx


def ag_group_gemm(a: torch.Tensor, b: torch.Tensor, ctx: MoEAgScatterGroupGemmContext, full_topk_ids: torch.Tensor,
                  sorted_output: bool = False):
    """``a`` [T/W, K] local tokens, ``b`` [E, N_local, K], ``full_topk_ids`` [T, k] (all ranks' routing) ->
    [T*k, N_local] in (token, slot) order, or the expert-sorted layout plus its ``MoESort`` when ``sorted_output``."""
    rt = ctx.rt
    W = ctx.num_ranks
    if not _native.use_native(a, b):
        full = ref_all_gather(a, rt.group) if W > 1 else a
        y = group_gemm_reference(full, b, full_topk_ids)
        if sorted_output:
            srt = sort_topk_ids_align_block_size(full_topk_ids, ctx.num_experts)
            ys = torch.zeros((srt.sorted_ids.numel(), y.shape[1]), dtype=y.dtype)
            ok = srt.sorted_ids >= 0
            ys[ok] = y[srt.sorted_ids[ok].long()]
            return ys, srt
        return y
    t_local = a.shape[0]
    if W > 1:
        buf = ctx.ag_buffer[:t_local * W]
        buf[ctx.rank * t_local:(ctx.rank + 1) * t_local].copy_(a)
        fast_allgather(buf, ctx.ag_ctx)
        full = buf
    else:
        full = a
    srt = sort_topk_ids_align_block_size(full_topk_ids, ctx.num_experts)
    ctx.last_sort = srt
    a_sorted = gather_sorted(full, srt)
    y_sorted = group_gemm_sorted(a_sorted, b, srt)
    if sorted_output:
        return y_sorted, srt
    return unsort(y_sorted, srt, full_topk_ids.numel())


# ------------------------------------------------------------------ grouped GEMM -> top-k reduce -> RS / AR
@dataclass
class MoEReduceRSContext:
    rt: Runtime
    rank: int
    world_size: int
    max_token_num: int
    hidden_dim: int
    num_experts: int
    topk: int
    dtype: torch.dtype
    rs_ctx: object = None
    ar_ctx: object = None

    def finalize(self):
        for c in (self.rs_ctx, self.ar_ctx):
            if c is not None:
                c.finalize()
        self.rs_ctx = self.ar_ctx = None


def create_moe_rs_context(rank: Optional[int] = None, world_size: Optional[int] = None,
                          local_world_size: Optional[int] = None, max_token_num: int = 0, hidden_dim: int = 0,
                          num_experts: int = 0, topk: int = 0, input_dtype: torch.dtype = torch.bfloat16,
                          n_chunks_max: int = 8) -> MoEReduceRSContext:
    rt = get_runtime()
    rank = rt.rank if rank is None else rank
    world_size = rt.world_size if world_size is None else world_size
    ctx = MoEReduceRSContext(rt, rank, world_size, max_token_num, hidden_dim, num_experts, topk, input_dtype)
    if rt.is_cuda and world_size > 1:
        ctx.rs_ctx = create_reduce_scater_2d_ctx(max_token_num, hidden_dim, dtype=input_dtype)
        ctx.ar_ctx = create_allreduce_ctx(max(4 * max_token_num * hidden_dim * 2, 1 << 20))
    return ctx


create_moe_ar_context = create_moe_rs_context


def _moe_down(x, weights, chosen_experts, expert_weight, ctx, srt: Optional[MoESort]):
    T = chosen_experts.shape[0]
    if not _native.use_native(x, weights):
        if srt is not None:   # x is in sorted layout: bring it back to (token, slot) order for the reference
            x = unsort(x, srt, chosen_experts.numel())
        return moe_reduce_reference(x, weights, chosen_experts, expert_weight)
    if srt is None:
        srt = sort_topk_ids_align_block_size(chosen_experts, ctx.num_experts)
        ids = srt.sorted_ids.long().clamp_min(0)
        xs = x[ids]
        xs[srt.sorted_ids < 0] = 0
        x = xs
    y_sorted = group_gemm_sorted(x, weights, srt)
    return reduce_topk(y_sorted, srt, expert_weight, T)


def run_moe_reduce_rs(x: torch.Tensor, weights: torch.Tensor, chosen_experts: torch.Tensor, expert_weight: torch.Tensor,
                      ctx: MoEReduceRSContext, n_chunks: int = 2, config=None, sort: Optional[MoESort] = None) -> torch.Tensor:
    """``x`` [T*k, I_local] ((token, slot) order, or expert-sorted when ``sort`` is given), ``weights`` [E, H, I_local]
    -> this rank's [T/W, H] block of ``sum_ranks sum_slots weight * (x @ w2^T)``."""
    part = _moe_down(x, weights, chosen_experts, expert_weight, ctx, sort)
    if ctx.world_size == 1:
        return part
    if not part.is_cuda:
        return ref_reduce_scatter(part, ctx.rt.group)
    return reduce_scatter_2d_op(part, ctx.rs_ctx)


def run_moe_reduce_ar(x: torch.Tensor, weights: torch.Tensor, chosen_experts: torch.Tensor, expert_weights: torch.Tensor,
                      ctx: MoEReduceRSContext, n_chunks: int = 4, config=None, sort: Optional[MoESort] = None) -> torch.Tensor:
    """Same as :func:`run_moe_reduce_rs` but every rank gets the full [T, H]."""
    part = _moe_down(x, weights, chosen_experts, expert_weights, ctx, sort)
    if ctx.world_size == 1:
        return part
    if not part.is_cuda:
        return ref_all_reduce(part, ctx.rt.group)
    return all_reduce(part, ctx=ctx.ar_ctx)

"""Tensor-parallel mixture-of-experts ops: router, token sort, grouped GEMM, AG -> grouped GEMM, grouped GEMM -> top-k
reduce -> reduce-scatter / all-reduce.

API of the reference: ``create_ag_group_gemm_context`` / ``ag_group_gemm`` (kernels/nvidia/allgather_group_gemm.py:337, :401),
``create_moe_rs_context`` / ``run_moe_reduce_rs`` (moe_reduce_rs.py:87, :710), ``run_moe_reduce_ar`` (moe_reduce_ar.py:482),
index helpers of moe_utils.py.  Expert weights are stored ``[E, N, K]`` (K-major rows, the layout the tcgen05 kernel
loads with TMA); the reference's ``[E, K, N]`` tensors are ``w.transpose(1, 2).contiguous()`` of these.

GPU path: ``csrc/moe.cu`` (router / sort / tile schedule / reduce) + ``csrc/moe_fused_sm100.cu``: ``ag_group_gemm`` is
ONE launch (comm CTAs push the tokens, the grouped tcgen05 GEMM gathers its A rows in the kernel and waits per row for
the chunk it needs, tiles visited in the device-computed arrival order); ``run_moe_reduce_rs`` / ``run_moe_reduce_ar``
are ONE launch (routing weight in the GEMM epilogue, N-chunk counters, reducer CTAs that top-k-sum finished chunks and
store them into the destination ranks' slots while later chunks compute).  CPU path and oracle: the torch restatements
below.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from .. import _native
from ..runtime import Runtime, get_runtime
from .common import new_ctx_dev, ref_all_gather, ref_all_reduce, ref_reduce_scatter, sm_count

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


def sort_topk_ids_staged(topk_ids: torch.Tensor, num_experts: int, tokens_per_rank: int, rank: int, world: int,
                         block_size: int = BLOCK_M) -> MoESort:
    """Like :func:`sort_topk_ids_align_block_size`, but inside an expert the rows are ordered by the ring distance
    ``(source rank - rank) mod world`` of their token, so that an expert's first tiles only need the token shards that
    arrive first during the fused all-gather (GPU: ``moe_align_sort_staged``; CPU: the same order in PyTorch)."""
    k = topk_ids.shape[-1]
    if _native.use_native(topk_ids):
        s, p, t, o, m, c = _native.load(True).moe_align_sort_staged(topk_ids.to(torch.int32).contiguous(), int(num_experts),
                                                                    int(block_size), int(k), int(tokens_per_rank), int(rank),
                                                                    int(world))
        return MoESort(s, p, t, o, m, c, k)
    base = sort_topk_ids_align_block_size(topk_ids, num_experts, block_size)
    ids = base.sorted_ids.clone()
    pos_of = base.pos_of.clone()
    offs = base.offsets.tolist()
    cnt = base.counts.tolist()
    for e in range(num_experts):
        rows = ids[offs[e]:offs[e] + cnt[e]]
        stage = ((rows // k) // tokens_per_rank - rank) % world
        rows = rows[torch.sort(stage, stable=True).indices]
        ids[offs[e]:offs[e] + cnt[e]] = rows
        pos_of[rows.long()] = torch.arange(offs[e], offs[e] + cnt[e], dtype=torch.int32)
    return MoESort(ids, pos_of, base.tile_expert, base.offsets, base.meta, base.counts, k)


def tile_schedule(srt: MoESort, tokens_per_rank: int, rank: int, world: int, block_size: int = BLOCK_M):
    """Device-side tile schedule ``(order, stage)`` of an expert-sorted layout (one 1024-thread CTA): the order the
    fused all-gather -> grouped GEMM visits the tiles in.  Same result as the host reference ``tile_arrival_order``
    (``csrc/moe_sched.cc``); the reference computes it with ``threadblock_swizzle_ag_moe`` kernels
    (threadblock_swizzle_ag_moe_triton.py:96-216, threadblock_swizzle_ag_moe.cu:248-413)."""
    if _native.use_native(srt.sorted_ids):
        order, stage, _ = _native.load(True).moe_tile_schedule(srt.sorted_ids, int(srt.k), int(tokens_per_rank), int(rank),
                                                               int(world), int(block_size))
        return order, stage
    return tile_arrival_order(srt, tokens_per_rank, rank, world, block_size)


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


def group_gemm_gather(x: torch.Tensor, w: torch.Tensor, srt: MoESort, a_row_div: int, scatter_out: bool = False,
                      row_weight: Optional[torch.Tensor] = None, order: Optional[torch.Tensor] = None,
                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Grouped GEMM whose A rows are gathered inside the kernel: sorted row r multiplies ``x[sorted_ids[r] // a_row_div]``
    (``a_row_div = k`` when ``x`` holds tokens, 1 when it holds (token, slot) pairs) with its tile's expert weight.
    Output in the sorted layout [cap, N], or in (token, slot) order [pairs, N] when ``scatter_out``; ``row_weight``
    [pairs] scales every row in the epilogue."""
    n_pairs = srt.pos_of.numel()
    rows = n_pairs if scatter_out else srt.sorted_ids.numel()
    if _native.use_native(x, w) and x.dtype == torch.bfloat16:
        if out is None:
            out = torch.empty((rows, w.shape[1]), dtype=x.dtype, device=x.device)
        rw = row_weight.reshape(-1).float().contiguous() if row_weight is not None else None
        _native.load(True).moe_group_gemm_gather(x, w.contiguous(), srt.sorted_ids, srt.tile_expert, order, srt.meta, out,
                                                 int(srt.k), int(a_row_div), bool(scatter_out), rw, 0)
        return out
    ids = srt.sorted_ids.long()
    ok = ids >= 0
    a = torch.zeros((ids.numel(), x.shape[1]), dtype=x.dtype, device=x.device)
    a[ok] = x[ids[ok] // a_row_div]
    y = group_gemm_sorted(a, w, srt).float()
    if row_weight is not None:
        y[ok] = y[ok] * row_weight.reshape(-1).float()[ids[ok]].unsqueeze(-1)
    y = y.to(x.dtype)
    if scatter_out:
        res = torch.zeros((rows, w.shape[1]), dtype=x.dtype, device=x.device)
        res[ids[ok]] = y[ok]
        y = res
    if out is not None:
        out.copy_(y)
        return out
    return y


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
    workspace: Optional[torch.Tensor] = None    # heap [2][max_ntokens][K]: the gathered tokens of the two call parities
    flags: Optional[torch.Tensor] = None        # heap [2][W][max_chunks] epoch flags, one per 128-token chunk
    ctx_dev: Optional[torch.Tensor] = None
    max_chunks: int = 0
    n_comm_ctas: int = 0                        # 0 = automatic
    last_sort: Optional[MoESort] = None
    last_order: Optional[torch.Tensor] = None

    @property
    def max_t_local(self) -> int:
        return self.max_ntokens // self.num_ranks

    def finalize(self):
        for n in ("workspace", "flags"):
            t = getattr(self, n)
            if t is not None:
                self.rt.symm_free(t)
                setattr(self, n, None)


def create_ag_group_gemm_context(max_ntokens: int, N_per_rank: int, K: int, num_experts: int, topk: int,
                                 dtype: torch.dtype = torch.bfloat16, rank: Optional[int] = None,
                                 num_ranks: Optional[int] = None, **kw) -> MoEAgScatterGroupGemmContext:
    rt = get_runtime()
    rank = rt.rank if rank is None else rank
    num_ranks = rt.world_size if num_ranks is None else num_ranks
    max_ntokens = (max_ntokens + num_ranks - 1) // num_ranks * num_ranks
    ctx = MoEAgScatterGroupGemmContext(rt, rank, num_ranks, max_ntokens, N_per_rank, K, num_experts, topk, dtype)
    if rt.is_cuda and num_ranks > 1:
        ctx.max_chunks = (ctx.max_t_local + BLOCK_M - 1) // BLOCK_M
        ctx.workspace = rt.symm_tensor((2, max_ntokens, K), dtype, zero=False, sync=False)
        ctx.flags = rt.symm_tensor((2, num_ranks, ctx.max_chunks), torch.int32, sync=False)
        ctx.ctx_dev = new_ctx_dev(rt)
        torch.cuda.synchronize()
        rt.host_barrier()
    return ctx


def ag_group_gemm(a: torch.Tensor, b: torch.Tensor, ctx: MoEAgScatterGroupGemmContext, full_topk_ids: torch.Tensor,
                  sorted_output: bool = False, sort: Optional[MoESort] = None):
    """``a`` [T/W, K] local tokens, ``b`` [E, N_local, K], ``full_topk_ids`` [T, k] (all ranks' routing) ->
    [T*k, N_local] in (token, slot) order, or the expert-sorted layout plus its ``MoESort`` when ``sorted_output``.

    GPU path: ONE launch (``moe_fused_sm100.cu``): comm CTAs push the local tokens to every rank with per-chunk flags,
    the grouped GEMM gathers its A rows inside the kernel, waiting per row for exactly the chunk it needs, and visits
    the tiles in the device-computed arrival order.  The routing is sorted once per call (``sort`` passes a sort made
    by the caller, e.g. shared with the down projection)."""
    rt = ctx.rt
    W = ctx.num_ranks
    if not _native.use_native(a, b):
        full = ref_all_gather(a, rt.group) if W > 1 else a
        y = group_gemm_reference(full, b, full_topk_ids)
        if sorted_output:
            srt = sort if sort is not None else sort_topk_ids_align_block_size(full_topk_ids, ctx.num_experts)
            ys = torch.zeros((srt.sorted_ids.numel(), y.shape[1]), dtype=y.dtype)
            ok = srt.sorted_ids >= 0
            ys[ok] = y[srt.sorted_ids[ok].long()]
            return ys, srt
        return y
    t_local = a.shape[0]
    if sort is not None:
        srt = sort
    elif W > 1:
        srt = sort_topk_ids_staged(full_topk_ids, ctx.num_experts, t_local, ctx.rank, W)
    else:
        srt = sort_topk_ids_align_block_size(full_topk_ids, ctx.num_experts)
    ctx.last_sort = srt
    if W == 1:
        y = group_gemm_gather(a, b, srt, a_row_div=srt.k, scatter_out=not sorted_output)
        return (y, srt) if sorted_output else y
    lib = _native.load(True)
    order, _stage = tile_schedule(srt, t_local, ctx.rank, W)
    ctx.last_order = order
    rows = srt.sorted_ids.numel() if sorted_output else full_topk_ids.numel()
    y = torch.empty((rows, b.shape[1]), dtype=a.dtype, device=a.device)
    n_sms = sm_count(a.device)
    n_comm = ctx.n_comm_ctas or max(4, min(16, 2 * (W - 1)))
    lib.moe_ag_group_gemm(rt.heap, a.contiguous(), b.contiguous(), srt.sorted_ids, srt.tile_expert, order, srt.meta, y,
                          int(srt.k), not sorted_output, ctx.workspace, ctx.flags, ctx.ctx_dev, ctx.max_t_local,
                          ctx.max_chunks, int(n_comm), n_sms, rt.config.wait_timeout_s)
    return (y, srt) if sorted_output else y


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
    n_chunks_max: int = 8
    n_red_ctas: int = 16                          # reducer CTAs of the fused launch
    rs_slots: Optional[torch.Tensor] = None      # heap [2][W][max_T / W][H]
    ar_slots: Optional[torch.Tensor] = None      # heap [2][W][max_T][H] (allocated on first all-reduce use)
    flags: Optional[torch.Tensor] = None         # heap [2][W][n_chunks_max * n_red]
    chunk_done: Optional[torch.Tensor] = None    # device [2][n_chunks_max]
    ctx_dev: Optional[torch.Tensor] = None
    y_sorted: Optional[torch.Tensor] = None      # scratch of the weighted expert outputs in the sorted layout

    def finalize(self):
        for n in ("rs_slots", "ar_slots", "flags"):
            t = getattr(self, n)
            if t is not None:
                self.rt.symm_free(t)
                setattr(self, n, None)


def create_moe_rs_context(rank: Optional[int] = None, world_size: Optional[int] = None,
                          local_world_size: Optional[int] = None, max_token_num: int = 0, hidden_dim: int = 0,
                          num_experts: int = 0, topk: int = 0, input_dtype: torch.dtype = torch.bfloat16,
                          n_chunks_max: int = 8, all_reduce: bool = False, n_red_ctas: int = 16) -> MoEReduceRSContext:
    """Slots, flags and chunk counters of the fused grouped GEMM -> top-k reduce -> reduce-scatter / all-reduce launch
    (collective call).  ``all_reduce`` also allocates the larger slots of the all-reduce form."""
    rt = get_runtime()
    rank = rt.rank if rank is None else rank
    world_size = rt.world_size if world_size is None else world_size
    max_token_num = (max_token_num + world_size - 1) // world_size * world_size
    ctx = MoEReduceRSContext(rt, rank, world_size, max_token_num, hidden_dim, num_experts, topk, input_dtype,
                             n_chunks_max=n_chunks_max, n_red_ctas=n_red_ctas)
    if rt.is_cuda and world_size > 1:
        W = world_size
        ctx.rs_slots = rt.symm_tensor((2, W, max_token_num // W, hidden_dim), input_dtype, zero=False, sync=False)
        if all_reduce:
            ctx.ar_slots = rt.symm_tensor((2, W, max_token_num, hidden_dim), input_dtype, zero=False, sync=False)
        ctx.flags = rt.symm_tensor((2, W, n_chunks_max * ctx.n_red_ctas), torch.int32, sync=False)
        ctx.chunk_done = torch.zeros(2 * n_chunks_max, dtype=torch.int32, device=rt.device)
        ctx.ctx_dev = new_ctx_dev(rt)
        torch.cuda.synchronize()
        rt.host_barrier()
    return ctx


def create_moe_ar_context(*args, **kw) -> MoEReduceRSContext:
    kw["all_reduce"] = True
    return create_moe_rs_context(*args, **kw)


def _moe_down_reference(x, weights, chosen_experts, expert_weight, srt: Optional[MoESort]):
    if srt is not None:   # x is in sorted layout: bring it back to (token, slot) order for the reference
        x = unsort(x, srt, chosen_experts.numel())
    return moe_reduce_reference(x, weights, chosen_experts, expert_weight)


def _moe_reduce_fused(x, weights, chosen_experts, expert_weight, ctx: MoEReduceRSContext, n_chunks: int,
                      srt: Optional[MoESort], all_reduce: bool) -> torch.Tensor:
    """One launch: grouped GEMM (rows gathered in the kernel, routing weight in the epilogue, N-chunk-major tile order
    with a counter per chunk) + reducer CTAs (top-k sum of finished chunks, P2P store into the destination slots, flags,
    final sum over the W slots).  Single GPU: the same GEMM with a local top-k reduce."""
    rt = ctx.rt
    W = ctx.world_size
    T, k = chosen_experts.shape
    H = weights.shape[1]
    x_sorted_layout = srt is not None
    if srt is None:
        srt = sort_topk_ids_align_block_size(chosen_experts, ctx.num_experts)
    # sorted-layout input: row r of x IS sorted row r (identity gather through an iota index); pair-order input: gather
    if x_sorted_layout:
        ids = srt.sorted_ids
        iota = torch.arange(ids.numel(), dtype=torch.int32, device=ids.device)
        gather_ids = torch.where(ids >= 0, iota, ids)
        w_rows = expert_weight.reshape(-1).float()[ids.clamp_min(0).long()]
        srt_g = MoESort(gather_ids, srt.pos_of, srt.tile_expert, srt.offsets, srt.meta, srt.counts, srt.k)
        row_weight = w_rows          # indexed by the gather id = sorted row
    else:
        srt_g = srt
        row_weight = expert_weight.reshape(-1).float().contiguous()
    cap = srt.sorted_ids.numel()
    if ctx.y_sorted is None or ctx.y_sorted.shape[0] < cap or ctx.y_sorted.shape[1] != H:
        ctx.y_sorted = torch.empty((cap, H), dtype=x.dtype, device=x.device)
    y_sorted = ctx.y_sorted[:cap]
    if W == 1:
        group_gemm_gather(x, weights, srt_g, a_row_div=1, scatter_out=False, row_weight=row_weight, out=y_sorted)
        return reduce_topk(y_sorted, srt, None, T)
    lib = _native.load(True)
    tiles_n = (H + 255) // 256
    n_chunks = max(1, min(int(n_chunks), ctx.n_chunks_max, tiles_n))
    if all_reduce and ctx.ar_slots is None:
        ctx.ar_slots = rt.symm_tensor((2, W, ctx.max_token_num, H), x.dtype, zero=False)
    slots = ctx.ar_slots if all_reduce else ctx.rs_slots
    out = torch.empty((T if all_reduce else T // W, H), dtype=x.dtype, device=x.device)
    lib.moe_group_gemm_reduce(rt.heap, x, weights.contiguous(), srt_g.sorted_ids, srt.tile_expert, srt.meta, y_sorted, int(k), 1,
                              row_weight, srt.pos_of, int(T), ctx.chunk_done, slots, ctx.flags, ctx.ctx_dev, out,
                              int(n_chunks), int(ctx.n_red_ctas), bool(all_reduce), sm_count(x.device),
                              rt.config.wait_timeout_s)
    return out


def run_moe_reduce_rs(x: torch.Tensor, weights: torch.Tensor, chosen_experts: torch.Tensor, expert_weight: torch.Tensor,
                      ctx: MoEReduceRSContext, n_chunks: int = 2, config=None, sort: Optional[MoESort] = None) -> torch.Tensor:
    """``x`` [T*k, I_local] ((token, slot) order, or expert-sorted when ``sort`` is given), ``weights`` [E, H, I_local]
    -> this rank's [T/W, H] block of ``sum_ranks sum_slots weight * (x @ w2^T)``.  ``n_chunks`` column chunks of the
    output are reduced and exchanged while the GEMM works on the next one."""
    if not _native.use_native(x, weights):
        part = _moe_down_reference(x, weights, chosen_experts, expert_weight, sort)
        return part if ctx.world_size == 1 else ref_reduce_scatter(part, ctx.rt.group)
    return _moe_reduce_fused(x, weights, chosen_experts, expert_weight, ctx, n_chunks, sort, all_reduce=False)


def run_moe_reduce_ar(x: torch.Tensor, weights: torch.Tensor, chosen_experts: torch.Tensor, expert_weights: torch.Tensor,
                      ctx: MoEReduceRSContext, n_chunks: int = 4, config=None, sort: Optional[MoESort] = None) -> torch.Tensor:
    """Same as :func:`run_moe_reduce_rs` but every rank gets the full [T, H]."""
    if not _native.use_native(x, weights):
        part = _moe_down_reference(x, weights, chosen_experts, expert_weights, sort)
        return part if ctx.world_size == 1 else ref_all_reduce(part, ctx.rt.group)
    return _moe_reduce_fused(x, weights, chosen_experts, expert_weights, ctx, n_chunks, sort, all_reduce=True)

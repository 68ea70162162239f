"""Expert-parallel all-to-all: dispatch (fp8 quantisation fused) and combine (top-k weighted sum fused).

API of the reference: ``create_all_to_all_context`` / ``fast_all_to_all`` / ``all_to_all_post_process``
(kernels/nvidia/low_latency_all_to_all.py:176, :198, :260) for the low-latency path and the dispatch / combine kernels
behind ``EPAll2AllLayer`` (kernels/nvidia/ep_a2a.py:38-447).  One context serves both layouts:

* ``layout="ll"``  fixed-stride receive areas ``[local expert][source rank][max tokens]``: no metadata exchange before
  the data (decode, low latency);
* ``layout="packed"``  receive rows packed per expert in (expert, source) order: per-expert counts are all-gathered with
  the low-latency packet all-gather first and every rank derives the exact offsets on the device (no CPU poll).

The receive side is turned into the expert-sorted, 128-row-aligned layout the grouped GEMM consumes
(:class:`EpRecv`), and ``ep_combine`` sends expert outputs back and reduces them with the routing weights.
CPU path / oracle: ``all_to_all`` emulation with torch.distributed.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from .. import _native
from ..runtime import Runtime, get_runtime
from .allgather import all_gather_ll, create_fast_allgather_context
from .common import new_ctx_dev
from .moe import MoESort, sort_topk_ids_align_block_size


@dataclass
class AllToAllContext:
    rt: Runtime
    max_m: int                 # tokens per rank
    hidden: int
    rank: int
    num_tot_experts: int
    world_size: int
    experts_per_rank: int
    topk: int
    dtype: torch.dtype
    quant: bool
    layout: str
    rows_per_parity: int = 0
    recv_x: Optional[torch.Tensor] = None
    recv_scale: Optional[torch.Tensor] = None
    recv_meta: Optional[torch.Tensor] = None
    recv_count: Optional[torch.Tensor] = None
    flags: Optional[torch.Tensor] = None
    ret: Optional[torch.Tensor] = None
    ret_flags: Optional[torch.Tensor] = None
    cursor: Optional[torch.Tensor] = None
    sent_row: Optional[torch.Tensor] = None
    dctx: Optional[torch.Tensor] = None      # dispatch call state
    cctx: Optional[torch.Tensor] = None      # combine call state
    counts_local: Optional[torch.Tensor] = None
    base: Optional[torch.Tensor] = None      # packed layout: [W][epr][W]
    ag_ctx: object = None

    def finalize(self):
        for t in (self.recv_x, self.recv_scale, self.recv_meta, self.recv_count, self.flags, self.ret, self.ret_flags):
            if t is not None:
                self.rt.symm_free(t)
        self.recv_x = None
        if self.ag_ctx is not None:
            self.ag_ctx.finalize()


@dataclass
class EpRecv:
    """What a rank holds after dispatch: rows sorted by local expert (padded to 128), ready for the grouped GEMM."""
    x_sorted: torch.Tensor          # [cap, H] bf16
    sort: MoESort                   # over receive rows (k = 1)
    recv_rows: int
    topk_ids: torch.Tensor          # the local routing that was dispatched (for combine)
    counts: Optional[torch.Tensor] = None   # [epr][W] tokens per (local expert, source)
    real_rows: Optional[torch.Tensor] = None   # packed list of the sorted rows that carry a token (+ their number)
    # CPU emulation only
    cpu_state: object = None


def create_all_to_all_context(max_m: int, hidden: int, rank: Optional[int] = None, num_tot_experts: int = 0,
                              world_size: Optional[int] = None, experts_per_rank: Optional[int] = None,
                              dtype: torch.dtype = torch.bfloat16, scale_dtype: torch.dtype = torch.float32, topk: int = 8,
                              quant: bool = True, layout: str = "ll") -> AllToAllContext:
    """Allocate the symmetric receive / return buffers (collective call)."""
    rt = get_runtime()
    rank = rt.rank if rank is None else rank
    world_size = rt.world_size if world_size is None else world_size
    epr = experts_per_rank if experts_per_rank is not None else num_tot_experts // world_size
    ctx = AllToAllContext(rt, max_m, hidden, rank, num_tot_experts, world_size, epr, topk, dtype, quant, layout)
    if not rt.is_cuda:
        return ctx
    W = world_size
    ctx.rows_per_parity = epr * W * max_m if layout == "ll" else W * max_m * topk
    row_bytes = hidden if quant else 2 * hidden
    ctx.recv_x = rt.symm_tensor((2, ctx.rows_per_parity, row_bytes), torch.uint8, zero=False)
    ctx.recv_scale = rt.symm_tensor((2, ctx.rows_per_parity, hidden // 128), torch.float32, zero=False)
    ctx.recv_meta = rt.symm_tensor((2, ctx.rows_per_parity), torch.int32, zero=False)
    ctx.recv_count = rt.symm_tensor((2, epr, W), torch.int32)
    ctx.flags = rt.symm_tensor((W,), torch.int32)
    ctx.ret = rt.symm_tensor((2, max_m * topk, hidden), torch.bfloat16, zero=False)
    ctx.ret_flags = rt.symm_tensor((W,), torch.int32)
    ctx.cursor = torch.zeros(num_tot_experts, dtype=torch.int32, device=rt.device)
    ctx.sent_row = torch.empty(max_m * topk, dtype=torch.int32, device=rt.device)
    ctx.dctx = new_ctx_dev(rt)
    ctx.cctx = new_ctx_dev(rt)
    if layout == "packed":
        ctx.counts_local = torch.zeros(num_tot_experts, dtype=torch.int32, device=rt.device)
        ctx.base = torch.zeros((W, epr, W), dtype=torch.int32, device=rt.device)
        ctx.ag_ctx = create_fast_allgather_context(max_ll_bytes=max(64 * 1024, 4 * num_tot_experts))
    torch.cuda.synchronize()
    rt.host_barrier()
    return ctx


# ------------------------------------------------------------------ CPU emulation (gloo) used as oracle
def _cpu_dispatch(ctx: AllToAllContext, x, topk_ids):
    rt, W, epr = ctx.rt, ctx.world_size, ctx.experts_per_rank
    T, k = topk_ids.shape
    send = [[] for _ in range(W)]
    for t in range(T):
        for j in range(k):
            e = int(topk_ids[t, j])
            if 0 <= e < ctx.num_tot_experts:
                send[e // epr].append((e % epr, t * k + j, x[t].clone()))
    gathered = [None] * W
    if W > 1:
        dist.all_gather_object(gathered, send, group=rt.cpu_group)
    else:
        gathered = [send]
    rows, experts, origin = [], [], []
    for src in range(W):
        for (le, pair, row) in gathered[src][ctx.rank]:
            rows.append(row)
            experts.append(le)
            origin.append((src, pair))
    n = len(rows)
    ids = torch.tensor(experts, dtype=torch.int32).reshape(-1, 1) if n else torch.zeros((0, 1), dtype=torch.int32)
    srt = sort_topk_ids_align_block_size(ids, epr)
    xs = torch.zeros((srt.sorted_ids.numel(), x.shape[1]), dtype=x.dtype)
    for r, sid in enumerate(srt.sorted_ids.tolist()):
        if sid >= 0:
            xs[r] = rows[sid]
    return EpRecv(xs, srt, n, topk_ids, cpu_state=origin)


def _cpu_combine(ctx: AllToAllContext, y_sorted, recv: EpRecv, topk_w):
    rt, W = ctx.rt, ctx.world_size
    back = [[] for _ in range(W)]
    pos = recv.sort.pos_of.tolist()
    for i, (src, pair) in enumerate(recv.cpu_state):
        back[src].append((pair, y_sorted[pos[i]].clone()))
    gathered = [None] * W
    if W > 1:
        dist.all_gather_object(gathered, back, group=rt.cpu_group)
    else:
        gathered = [back]
    T, k = recv.topk_ids.shape
    out = torch.zeros((T, y_sorted.shape[1]), dtype=torch.float32)
    for src in range(W):
        for (pair, row) in gathered[src][ctx.rank]:
            w = float(topk_w.reshape(-1)[pair]) if topk_w is not None else 1.0
            out[pair // k] += w * row.float()
    return out.to(y_sorted.dtype)


def _parts_for_rows(rows: int) -> int:
    """Warps that share one row.  Moving a row is a chain of dependent memory round trips; a decode step has few rows,
    so several warps per row cut the latency, while a prefill-sized batch keeps one warp per row for throughput."""
    return 4 if rows <= 1024 else 2 if rows <= 2048 else 1


def _ctas_for_rows(rows: int, parts: int = 1) -> int:
    """Eight warps per CTA, ``parts`` warps per row: at least 64 CTAs for a decode step, up to four per SM for
    prefill-sized batches."""
    return int(min(592, max(64, rows * parts // 8)))


# ------------------------------------------------------------------ public ops
def ep_dispatch(ctx: AllToAllContext, x: torch.Tensor, topk_ids: torch.Tensor) -> EpRecv:
    """Send every (token, slot) to the rank owning its expert; returns the local expert-sorted receive view."""
    if not _native.use_native(x):
        return _cpu_dispatch(ctx, x, topk_ids)
    lib = _native.load(True)
    rt, W, epr, E = ctx.rt, ctx.world_size, ctx.experts_per_rank, ctx.num_tot_experts
    ids = topk_ids.to(torch.int32).contiguous()
    base = None
    base_self = None
    if ctx.layout == "packed":
        lib.ep_count(ids, E, ctx.counts_local)
        counts_all = all_gather_ll(ctx.counts_local, ctx.ag_ctx) if W > 1 else ctx.counts_local.unsqueeze(0)
        lib.ep_layout(counts_all.contiguous(), ctx.base, epr, W, E)
        base = ctx.base
        base_self = ctx.base[ctx.rank].reshape(-1)
    parts = _parts_for_rows(ids.numel())
    lib.ep_dispatch(rt.heap, x.contiguous(), ids, E, ctx.quant, ctx.max_m, ctx.recv_x, ctx.recv_scale, ctx.recv_meta,
                    ctx.recv_count, ctx.flags, ctx.rows_per_parity, base, ctx.cursor, ctx.sent_row, ctx.dctx,
                    _ctas_for_rows(ids.numel(), parts), rt.config.wait_timeout_s, parts)
    # Receive side, one launch: the receive areas are grouped by (expert, source) already, so the grouped-GEMM layout
    # (rows sorted by local expert, 128-row padding) follows from the epr x W counts; fp8 rows are de-quantised while
    # they are moved.  sorted_ids index receive rows; nothing scans the receive capacity.
    cap = min(ctx.rows_per_parity, W * ctx.max_m * max(ctx.topk, ids.shape[1])) + epr * 127
    cap = (cap + 127) // 128 * 128
    xs, sid, tile_expert, offsets, meta, counts, real_rows = lib.ep_finish(
        ctx.recv_x, ctx.recv_scale, ctx.recv_count, base_self, epr, W, ctx.max_m, ctx.hidden, ctx.quant, ctx.rows_per_parity,
        ctx.dctx, cap, _ctas_for_rows(min(cap, W * ids.numel()), parts), parts)
    srt = MoESort(sid, None, tile_expert, offsets, meta, counts, 1)
    return EpRecv(xs, srt, ctx.rows_per_parity, ids, counts=ctx.recv_count, real_rows=real_rows)


def ep_combine(ctx: AllToAllContext, y_sorted: torch.Tensor, recv: EpRecv, topk_w: Optional[torch.Tensor]) -> torch.Tensor:
    """Return expert outputs (sorted layout) to their tokens and take the weighted sum over the k slots -> [T, H]."""
    if not _native.use_native(y_sorted):
        return _cpu_combine(ctx, y_sorted, recv, topk_w)
    lib = _native.load(True)
    rt = ctx.rt
    base_self = ctx.base[ctx.rank].reshape(-1) if ctx.layout == "packed" else None
    w = topk_w.float().contiguous() if topk_w is not None else None
    parts = _parts_for_rows(recv.topk_ids.numel())
    return lib.ep_combine(rt.heap, y_sorted.contiguous(), recv.sort.pos_of, ctx.recv_meta, ctx.dctx, base_self, ctx.max_m,
                          ctx.rows_per_parity, ctx.ret, ctx.ret_flags, recv.topk_ids, w, ctx.num_tot_experts, ctx.cctx,
                          _ctas_for_rows(recv.topk_ids.numel(), parts), rt.config.wait_timeout_s,
                          recv.sort.sorted_ids, recv.sort.meta, recv.real_rows, parts)


def fast_all_to_all(ctx: AllToAllContext, send_tensor: torch.Tensor, send_split_cumsum: torch.Tensor,
                    send_scale: Optional[torch.Tensor] = None) -> EpRecv:
    """Reference-style entry: ``send_tensor`` rows are already sorted by global expert and ``send_split_cumsum`` [E+1]
    gives the row range of every expert.  Equivalent to a dispatch with one slot per row."""
    E = ctx.num_tot_experts
    cs = send_split_cumsum.to(torch.int64)
    n = send_tensor.shape[0]
    rows = torch.arange(n, device=send_tensor.device)
    ids = (torch.searchsorted(cs[1:].contiguous(), rows, right=True)).to(torch.int32).reshape(n, 1)
    ids = torch.where(rows.reshape(n, 1) < cs[-1], ids, torch.full_like(ids, E))
    return ep_dispatch(ctx, send_tensor, ids)


def all_to_all_post_process(ctx: AllToAllContext, recv: EpRecv) -> Tuple[torch.Tensor, torch.Tensor]:
    """Compact view of a receive: (rows sorted by local expert without padding, tokens per local expert)."""
    sid = recv.sort.sorted_ids
    keep = sid >= 0
    return recv.x_sorted[keep], recv.sort.counts


def fp8_quant(x: torch.Tensor):
    """Per-row, per-128-element e4m3 quantisation: returns (fp8 [T,H], fp32 scales [T,H/128]); scale = amax / 448."""
    if _native.use_native(x) and x.dtype == torch.bfloat16 and x.shape[-1] % 128 == 0:
        return _native.load(True).fp8_quant(x.contiguous())
    T, H = x.shape
    xb = x.float().reshape(T, H // 128, 128)
    s = xb.abs().amax(-1).clamp_min(1e-10) / 448.0
    q = (xb / s.unsqueeze(-1)).reshape(T, H).to(torch.float8_e4m3fn)
    return q, s


def fp8_dequant(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    if _native.use_native(q):
        return _native.load(True).fp8_dequant(q.contiguous(), s.contiguous())
    T, H = q.shape
    return (q.float().reshape(T, H // 128, 128) * s.unsqueeze(-1)).reshape(T, H).to(torch.bfloat16)

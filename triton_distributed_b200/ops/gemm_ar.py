"""Decode-size GEMM (M <= 256) with split-K, and GEMM -> AllReduce in one launch.

API of the reference: ``create_gemm_ar_context`` / ``create_ll_gemm_ar_context`` / ``gemm_allreduce_op`` /
``low_latency_gemm_allreduce_op`` (python/triton_dist/kernels/nvidia/gemm_allreduce.py:94, :111, :546, :509).
Inputs ``a`` [M, K/W], ``b`` [N, K/W] (row-parallel weight, K-major) -> ``[M, N]`` summed over the ranks.

GPU path: ``csrc/gemm_ar_sm100.cu`` (swap-AB tcgen05 kernel; the last split-K CTA of every 128-column tile runs that
tile's cross-rank sum through NVLS ``multimem.ld_reduce`` or peer stores).  For M > 256 the op falls back to the
large-tile GEMM followed by the all-reduce library.  CPU / reference path: ``matmul`` + ``all_reduce``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from .. import _native
from ..runtime import Runtime, get_runtime
from ..tools.autotuner import current_config
from ..utils.oplog import logged_op
from .common import new_ctx_dev, ref_all_reduce, sm_count

MAX_SKINNY_M = 256
# Exchange of the split-K parts inside a cluster: "ld" = the reducing CTA loads its rows from the peers' shared memory,
# "bulk" = every CTA sends each peer its rows with one bulk copy.  TDB200_SKINNY_EXCHANGE overrides.
SKINNY_EXCHANGE = "ld"


def _bulk_exchange() -> int:
    import os
    return 1 if os.environ.get("TDB200_SKINNY_EXCHANGE", SKINNY_EXCHANGE) == "bulk" else 0

_SCRATCH: Dict[Tuple[int, int], Tuple[torch.Tensor, torch.Tensor]] = {}
_UNFIT_TABLE_SHAPES: set = set()   # (token pad, N, K, tile width, cluster size) from the tuned table that did not fit here


def _scratch(device, need_acc: int, need_tiles: int):
    """Per-device split-K scratch (fp32 accumulator + tile counters); the kernel leaves both zeroed."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), 0)
    cur = _SCRATCH.get(key)
    if cur is None or cur[0].numel() < need_acc or cur[1].numel() < need_tiles:
        acc = torch.zeros(max(need_acc, 1 << 20), dtype=torch.float32, device=device)
        cnt = torch.zeros(max(need_tiles, 4096), dtype=torch.int32, device=device)
        _SCRATCH[key] = (acc, cnt)
        cur = _SCRATCH[key]
    return cur


def _mpad(m: int) -> int:
    return 16 if m <= 16 else 32 if m <= 32 else 64 if m <= 64 else 128 if m <= 128 else 256


def split_scratch_elems(m: int, n: int) -> int:
    """fp32 elements of the stream-K form's accumulation buffer for up to ``m`` tokens and ``n`` columns: column-major
    [ceil(n / 128) * 128][token pad], so that a thread's consecutive tokens are contiguous (vector reductions)."""
    return (n + 127) // 128 * 128 * _mpad(m)


def cluster_config(M: int, N: int, K: int) -> Tuple[int, int]:
    """(tile width in 128-column blocks, CTAs per tile) of the cluster form for this problem: what the autotuner is
    trying, else the measured winner from ``ops.tuned_configs``, else (0, 0) = the launcher's cost model."""
    tuned = current_config()
    if "cluster_nt" in tuned and "cluster_s" in tuned:
        return int(tuned["cluster_nt"]), int(tuned["cluster_s"])
    from .tuned_configs import lookup, lookup_user
    cfg = lookup_user("skinny_gemm", 1, _mpad(M), N, K)
    if cfg is None and sm_count(torch.cuda.current_device()) == 148:   # the built-in table was measured on 148 SMs
        cfg = lookup("skinny_gemm", 1, _mpad(M), N, K)
    return (int(cfg["cluster_nt"]), int(cfg["cluster_s"])) if cfg else (0, 0)


def _rows_aligned(t: torch.Tensor, nbytes: int) -> bool:
    """Whether every row of the 2-D tensor starts on an ``nbytes`` boundary."""
    return t.data_ptr() % nbytes == 0 and (t.stride(0) * t.element_size()) % nbytes == 0


def skinny_gemm(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, splits: int = 0,
                cluster: Optional[Tuple[int, int]] = None) -> torch.Tensor:
    """``x`` [M<=256, K] @ ``w`` [N, K]^T with the weight-streaming kernel.  ``splits`` >= 1 asks for the stream-K form
    with about that many pieces per column tile; 0 runs the cluster form where it fits.  ``cluster`` = (tile width in
    128-column blocks, CTAs per tile) fixes the cluster form's shape (an infeasible one raises)."""
    lib = _native.load(True)
    M, K = x.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    acc, cnt = _scratch(x.device, split_scratch_elems(M, N), (N + 127) // 128)
    if splits < 1 and not _rows_aligned(out, 8):
        # the cluster form stores four bf16 values at a time: an output view whose rows do not start on 8-byte boundaries
        # goes through the stream-K form, which stores single values
        if cluster is not None and cluster[0] >= 1:
            raise ValueError("skinny_gemm: the cluster form needs output rows that start on 8-byte boundaries")
        splits, cluster = max(1, pick_stream_k_splits(M, N, K)), None
    nt, s = cluster if cluster is not None else (cluster_config(M, N, K) if splits < 1 else (0, 0))
    if cluster is None and (_mpad(M), N, K, nt, s) in _UNFIT_TABLE_SHAPES:
        nt, s = 0, 0
    try:
        lib.skinny_gemm_bf16(x, w, out, acc, cnt, splits, 0, nt, s, _bulk_exchange())
    except RuntimeError:
        # a shape from the tuned table that this GPU cannot hold in one wave of clusters (the SMs per GPC differ from
        # part to part) is a hint, not a demand: remember it and let the launcher choose.  The refusal happens on the
        # host before anything is launched.
        if cluster is not None or (nt, s) == (0, 0):
            raise
        _UNFIT_TABLE_SHAPES.add((_mpad(M), N, K, nt, s))
        lib.skinny_gemm_bf16(x, w, out, acc, cnt, splits, 0, 0, 0, _bulk_exchange())
    return out


@dataclass
class GemmARContext:
    rt: Runtime
    rank: int
    world_size: int
    max_M: int
    N: int
    dtype: torch.dtype
    m_cap: int = 0
    use_multimem: bool = True
    partial: Optional[torch.Tensor] = None   # heap
    flags: Optional[torch.Tensor] = None     # heap [W][max_tiles]
    acc: Optional[torch.Tensor] = None
    counters: Optional[torch.Tensor] = None
    ctx_dev: Optional[torch.Tensor] = None
    max_tiles: int = 0
    ar_ctx: object = None                    # all-reduce library context for the large-M path
    calls: int = 0
    splits: Optional[int] = None             # K splits per column tile: None = by M (see pick_gemm_ar_splits)

    def finalize(self):
        if self.partial is not None:
            self.rt.symm_free(self.partial)
            self.rt.symm_free(self.flags)
            self.partial = None
        if self.ar_ctx is not None:
            self.ar_ctx.finalize()
            self.ar_ctx = None


LLGemmARContext = GemmARContext


def create_gemm_ar_context(ar_stream=None, rank: Optional[int] = None, world_size: Optional[int] = None,
                           local_world_size: Optional[int] = None, max_M: int = 256, N: int = 0,
                           dtype: torch.dtype = torch.bfloat16, MIN_BLOCK_SIZE_M: int = 16, MIN_BLOCK_SIZE_N: int = 16,
                           NUM_COMM_SMS: int = 132, use_multimem: bool = True) -> GemmARContext:
    """Allocate the heap partial-tile buffer and per-tile flags (collective call)."""
    from .allreduce import create_allreduce_ctx

    rt = get_runtime()
    rank = rt.rank if rank is None else rank
    world_size = rt.world_size if world_size is None else world_size
    import os
    # The push form (each rank stores its partial tile into every peer's slot: one NVLink latency) beat the NVLS form
    # (flag, then multimem.ld_reduce: two latencies) by 2-10 % on two ranks at every size, and by 9 % on four ranks at
    # 16 tokens (29.9 against 32.5 us); from 64 tokens on four ranks the switch's sum wins (36.6 against 38.7 us).  The
    # form is a property of the context (the partial buffers differ), so it follows the context's token capacity.
    # TDB200_GEMM_AR_MC=0 / 1 forces one form.
    mc_env = os.environ.get("TDB200_GEMM_AR_MC", "")
    if mc_env in ("0", "1"):
        use_multimem = mc_env == "1"
    elif world_size == 2 or max_M <= 32:
        use_multimem = False
    ctx = GemmARContext(rt=rt, rank=rank, world_size=world_size, max_M=max_M, N=N, dtype=dtype,
                        use_multimem=use_multimem)
    if rt.is_cuda and world_size > 1:
        ctx.m_cap = min(max_M, MAX_SKINNY_M)
        ctx.max_tiles = (N + 127) // 128
        slots = 1 if (use_multimem and rt.has_multicast) else world_size
        ctx.partial = rt.symm_tensor((2, slots, ctx.m_cap, N), dtype, zero=False)
        ctx.flags = rt.symm_tensor((world_size, ctx.max_tiles), torch.int32)
        ctx.acc = torch.zeros(split_scratch_elems(ctx.m_cap, N), dtype=torch.float32, device=rt.device)
        ctx.counters = torch.zeros(ctx.max_tiles, dtype=torch.int32, device=rt.device)
        ctx.ctx_dev = new_ctx_dev(rt)
        if max_M > MAX_SKINNY_M:
            ctx.ar_ctx = create_allreduce_ctx(max(4 * max_M * N * 2, 1 << 20))
        torch.cuda.synchronize()
        rt.host_barrier()
    return ctx


def create_ll_gemm_ar_context(rank: Optional[int] = None, world_size: Optional[int] = None,
                              local_world_size: Optional[int] = None, max_M: int = 256, N: int = 0,
                              dtype: torch.dtype = torch.bfloat16, MIN_BLOCK_SIZE_M: int = 16,
                              MIN_BLOCK_SIZE_N: int = 16, NUM_COMM_SMS: int = 16, num_phases: int = 2) -> GemmARContext:
    return create_gemm_ar_context(None, rank, world_size, local_world_size, max_M, N, dtype)


def pick_gemm_ar_splits(M: int, N: int = 5120, K: int = 3200, num_sms: int = 148) -> int:
    """K splits per 128-column tile of the swap-AB kernel; 0 leaves the choice to the launcher, which then runs the
    cluster form (the CTAs of a thread-block cluster split one tile's K range and sum their parts through distributed
    shared memory) wherever the tiles fit into one wave of clusters.  With ``TDB200_SKINNY_FORM=1`` (stream-K form
    only): up to 16 tokens the weights are everything and the stream-K partition over all SMs (0) wins; from 32 tokens
    on the fp32 split accumulation (M x 128 atomics per piece, then a read-back by the last arriver) costs more than
    idle SMs, so a tile is computed whole by one CTA and goes straight to its bf16 destination - unless K is so long
    (more than 64 k-blocks per CTA) that the few CTAs would stream for too long; then K is split as far as the SM
    count allows.  ``TDB200_GEMM_AR_SPLITS`` overrides."""
    import os
    v = os.environ.get("TDB200_GEMM_AR_SPLITS")
    if v not in (None, ""):
        return int(v)
    if os.environ.get("TDB200_SKINNY_FORM", "0") != "1":
        return 0
    return pick_stream_k_splits(M, N, K, num_sms)


def pick_stream_k_splits(M: int, N: int, K: int, num_sms: int = 148) -> int:
    """Split count of the stream-K form (see :func:`pick_gemm_ar_splits`)."""
    if M <= 16:
        return 0
    tiles = (N + 127) // 128
    kb = (K + 63) // 64
    return max(1, min(num_sms // max(tiles, 1), -(-kb // 64)))


def gemm_ar_reference(a: torch.Tensor, b: torch.Tensor, group=None) -> torch.Tensor:
    return ref_all_reduce(torch.matmul(a, b.t()), group)


def _gemm_ar_meta(ctx, a, b, *args, **kw):
    M, K = a.shape
    N = b.shape[0]
    W = ctx.world_size
    return {"shape": {"M": M, "N": N, "K": K * W, "world": W}, "flops": 2.0 * M * N * K,
            "link_bytes": 2.0 * (W - 1) / max(W, 1) * M * N * a.element_size()}


@logged_op("gemm_allreduce", _gemm_ar_meta)
def gemm_allreduce_op(ctx: GemmARContext, a: torch.Tensor, b: torch.Tensor, cfg=None, output: Optional[torch.Tensor] = None,
                      straggler_option=None) -> torch.Tensor:
    """``a`` [M, K_local] @ ``b`` [N, K_local]^T summed over ranks -> [M, N] on every rank."""
    rt = ctx.rt
    if not _native.use_native(a, b) or a.dtype != torch.bfloat16:
        res = gemm_ar_reference(a, b, rt.group)
        if output is not None:
            output.copy_(res)
            return output
        return res
    lib = _native.load(True)
    M, K = a.shape
    N = b.shape[0]
    if output is None:
        output = torch.empty((M, N), dtype=a.dtype, device=a.device)
    if a.stride(-1) != 1:
        a = a.contiguous()
    if ctx.world_size == 1:
        from .gemm import gemm
        if M <= MAX_SKINNY_M:
            return skinny_gemm(a, b, out=output)
        return gemm(a, b, out=output)
    if M > ctx.m_cap:
        from .allreduce import all_reduce
        from .gemm import gemm
        part = gemm(a, b)
        return all_reduce(part, ctx=ctx.ar_ctx, output=output)
    if N != ctx.N:
        raise ValueError(f"gemm_allreduce_op: N={N} differs from the context's N={ctx.N}")
    tuned = current_config()
    splits = tuned["gemm_ar_splits"] if "gemm_ar_splits" in tuned else (
        ctx.splits if ctx.splits is not None else pick_gemm_ar_splits(M, N, K))
    final = None
    if not _rows_aligned(output, 16):
        # the cross-rank sum stores 16 bytes at a time: a misaligned output view is filled through an aligned buffer
        final, output = output, torch.empty((M, N), dtype=a.dtype, device=a.device)
    nt, s = 0, 0          # the launcher's choice: in all-reduce mode always 128-column tiles (one exchange per cluster)
    tuned_now = current_config()
    if "cluster_nt" in tuned_now and "cluster_s" in tuned_now and int(splits) < 1:
        nt, s = int(tuned_now["cluster_nt"]), int(tuned_now["cluster_s"])
    lib.gemm_ar_bf16(rt.heap, a, b, output, ctx.acc, ctx.counters, ctx.partial, ctx.flags, ctx.ctx_dev, ctx.m_cap,
                     ctx.max_tiles, int(splits), 0, bool(ctx.use_multimem), rt.config.wait_timeout_s, nt, s,
                     _bulk_exchange())
    ctx.calls += 1
    if final is not None:
        final.copy_(output)
        return final
    return output


low_latency_gemm_allreduce_op = gemm_allreduce_op

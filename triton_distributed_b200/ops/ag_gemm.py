"""AllGather -> GEMM in one kernel launch (``ag_gemm``).

API of the reference: ``create_ag_gemm_context`` / ``ag_gemm``
(python/triton_dist/kernels/nvidia/allgather_gemm.py:489, :534).  Inputs: ``a`` [M/W, K] (rows sharded over the
ranks), ``b`` [N/W, K] (column-parallel weight, K-major); output [M, N/W].

GPU path: ``csrc/gemm_sm100.cu`` in all-gather mode - comm CTAs of the launch push the local shard into
every rank's workspace with bulk-TMA copies (or NVLS ``multimem.st``) and set per-chunk epoch flags; the
tcgen05 GEMM CTAs wait for exactly the chunk a tile needs and compute the local shard first.
CPU / reference path: ``all_gather_into_tensor`` + ``matmul`` (what the reference's ``torch_ag_gemm`` does,
layers/nvidia/tp_mlp.py:231-242).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Optional, Tuple

import torch

from .. import _native
from ..runtime import Runtime, get_runtime
from ..tools.autotuner import config_space, contextual_autotune, current_config
from ..utils.oplog import logged_op
from .gemm import use_cta_pair
from .common import new_ctx_dev, ref_all_gather, sm_count

BLOCK_M = 128


@dataclass
class AllGatherGEMMTensorParallelContext:
    rt: Runtime
    rank: int
    num_ranks: int
    max_M: int                 # global rows the workspace can hold
    K: int
    dtype: torch.dtype
    BLOCK_N: int = 256
    kernel_form: str = "auto"   # "auto" | "single" (128 x BLOCK_N tiles) | "pair" (256 x 256 tiles over two SMs)
    n_comm_ctas: int = 0       # 0 = automatic
    num_ctas: int = 0
    use_multimem: bool = False
    mc_explicit: bool = False  # the caller (or the environment) chose the push flavour: the tuned table does not override it
    for_correctness: bool = False
    workspace: Optional[torch.Tensor] = None   # heap [2][max_M][K]
    flags: Optional[torch.Tensor] = None       # heap [2][W][max_chunks]
    ctx_dev: Optional[torch.Tensor] = None
    max_chunks: int = 0
    calls: int = 0
    stats: Optional[torch.Tensor] = None       # optional int64 [num_ctas, 8] stall counters filled by the pair kernel

    @property
    def max_seg_rows(self) -> int:
        return self.max_M // self.num_ranks

    def finalize(self):
        if self.workspace is not None:
            self.rt.symm_free(self.workspace)
            self.rt.symm_free(self.flags)
            self.workspace = None
            self.flags = None


def create_ag_gemm_context(tensor_A: Optional[torch.Tensor] = None, tensor_B: Optional[torch.Tensor] = None,
                           rank: Optional[int] = None, num_ranks: Optional[int] = None, max_M: Optional[int] = None,
                           num_local_ranks: int = 8, BLOCK_M: int = 128, BLOCK_N: int = 256, BLOCK_K: int = 64,
                           stages: int = 3, ag_intranode_stream=None, ag_internode_stream=None,
                           for_correctness: bool = False, K: Optional[int] = None, dtype: Optional[torch.dtype] = None,
                           n_comm_ctas: int = 0, use_multimem: Optional[bool] = None) -> AllGatherGEMMTensorParallelContext:
    """Allocate the symmetric workspace and flags (collective call: every rank, same arguments).

    ``max_M`` is the gathered row count (``world * rows_per_rank``).  Stream / tile arguments of the
    reference signature are accepted and ignored: the all-gather runs inside the GEMM launch and the tile
    shape is fixed by the tcgen05 kernel (128 x BLOCK_N x 64).
    """
    rt = get_runtime()
    rank = rt.rank if rank is None else rank
    num_ranks = rt.world_size if num_ranks is None else num_ranks
    if tensor_A is not None:
        K = tensor_A.shape[-1] if K is None else K
        dtype = tensor_A.dtype if dtype is None else dtype
        if max_M is None:
            max_M = tensor_A.shape[0] * num_ranks
    if K is None or max_M is None:
        raise ValueError("create_ag_gemm_context needs tensor_A or (max_M, K)")
    dtype = dtype or torch.bfloat16
    max_M = (max_M + num_ranks - 1) // num_ranks * num_ranks
    import os
    mc_explicit = use_multimem is not None or "TDB200_AG_MULTIMEM" in os.environ
    if use_multimem is None:
        # From four ranks on the NVLS push wins: every byte leaves the GPU once instead of W - 1 times, so four comm
        # CTAs carry the whole all-gather; between two ranks there is nothing to replicate.
        use_multimem = num_ranks >= 4 and os.environ.get("TDB200_AG_MULTIMEM", "1") != "0"
    ctx = AllGatherGEMMTensorParallelContext(rt=rt, rank=rank, num_ranks=num_ranks, max_M=max_M, K=K, dtype=dtype,
                                             BLOCK_N=BLOCK_N if BLOCK_N in (128, 256) else 256,
                                             n_comm_ctas=n_comm_ctas, use_multimem=use_multimem,
                                             mc_explicit=mc_explicit, for_correctness=for_correctness)
    if rt.is_cuda and num_ranks > 1:
        # flag words per source: one per 128-row chunk for the unicast push, one per (chunk, comm CTA <= 8) for NVLS
        ctx.max_chunks = 8 * ((ctx.max_seg_rows + BLOCK_M - 1) // BLOCK_M)
        ctx.workspace = rt.symm_tensor((2, max_M, K), dtype, zero=False)
        ctx.flags = rt.symm_tensor((2, num_ranks, ctx.max_chunks), torch.int32)
        ctx.ctx_dev = new_ctx_dev(rt)
        torch.cuda.synchronize()
        rt.host_barrier()
    return ctx


PUSH_GBS_PER_CTA = 22.0     # effective rate of one bulk-TMA comm CTA while the GEMM runs (ten of them starved the
                            # eight-rank GEMM for a third of its time, twenty did not)
LINK_GBS = 770.0            # measured peer-copy bandwidth per direction
PAIR_TILE_TFLOPS = 20.5     # measured: one CTA pair sustains about 20.5 TFLOP/s on 256 x 256 tiles


def pair_wave_time(tiles: int, pairs: int) -> float:
    """Duration of a pair-kernel GEMM in tile times: full waves, and an incomplete last wave that costs half a tile
    when it occupies at most half the pairs (its tiles are then computed as two 128-column halves)."""
    full, rem = divmod(tiles, pairs)
    if rem == 0:
        return float(full)
    return full + (0.5 if 2 * rem <= pairs else 1.0)


def pick_comm_ctas(rows_per_rank: int, n_local: int, world: int, block_n: int, n_sms: int, pair: bool = False,
                   k: int = 8192) -> int:
    """Comm CTAs of the fused launch.  Every comm CTA is an SM the GEMM does not get, so the count is the smallest
    one whose push bandwidth keeps the remote shards ahead of the GEMM (rank distance d's shard is needed after d
    segments of GEMM time), unless taking more SMs away does not lengthen the GEMM's wave count anyway.  With the
    CTA-pair kernel the work units are 256 x 256 tiles on SM pairs and the count is even."""
    n_floor = 2 if world <= 2 else 4
    if pair:
        tiles_seg = ((rows_per_rank + 2 * BLOCK_M - 1) // (2 * BLOCK_M)) * ((n_local + 255) // 256)
        tiles = world * tiles_seg
        tile_us = 2.0 * 256 * 256 * k / (PAIR_TILE_TFLOPS * 1e6)
        shard_mb = rows_per_rank * k * 2 / 1e6
        best, best_t = n_floor, None
        for n in range(n_floor, 34, 2):
            pairs = (n_sms - n) // 2
            if pairs < 1:
                break
            gemm_us = pair_wave_time(tiles, pairs) * tile_us
            seg_us = gemm_us / world
            push_gbs = min(n * PUSH_GBS_PER_CTA, LINK_GBS)
            # shard d (d = 1 .. world-1) has arrived after d * shard / rate and is needed after d * seg_us
            stall_us = max(0.0, (world - 1) * (shard_mb * 1e3 / push_gbs - seg_us)) if world > 1 else 0.0
            t = gemm_us + stall_us
            if best_t is None or t < best_t - 1e-9:
                best, best_t = n, t
        return int(best)
    n_min = 4 if world <= 2 else 8
    tiles = world * ((rows_per_rank + BLOCK_M - 1) // BLOCK_M) * ((n_local + block_n - 1) // block_n)
    waves = max(1, -(-tiles // (n_sms - n_min)))
    n_gemm = -(-tiles // waves)
    return int(max(n_min, min(32, n_sms - n_gemm)))


def ag_gemm_reference(a: torch.Tensor, b: torch.Tensor, group=None) -> torch.Tensor:
    """all_gather(a) @ b^T with torch.distributed + torch.matmul."""
    return torch.matmul(ref_all_gather(a, group), b.t())


def _ag_meta(a, b, ctx, *args, **kw):
    W = ctx.num_ranks
    m, K = a.shape
    N = b.shape[0]
    return {"shape": {"M": m * W, "N": N, "K": K, "world": W}, "flops": 2.0 * m * W * N * K,
            "link_bytes": (W - 1) * m * K * a.element_size()}


# candidates of the contextual autotuner: launch-level knobs of the fused kernel
AG_GEMM_TUNE_SPACE = (config_space(use_multimem=[False], n_comm_ctas=[4, 8, 12, 16, 20]) +
                      config_space(use_multimem=[True], n_comm_ctas=[2, 4, 8]))


@contextual_autotune(configs=AG_GEMM_TUNE_SPACE, is_dist=True,
                     key=lambda a, b, ctx, **kw: f"W{ctx.num_ranks}_m{a.shape[0]}_N{b.shape[0]}_K{a.shape[1]}")
def _ag_gemm_tuned(a, b, ctx, **kw):
    return ag_gemm(a, b, ctx, autotune=False, **kw)


@logged_op("ag_gemm", _ag_meta)
def ag_gemm(a: torch.Tensor, b: torch.Tensor, ctx: AllGatherGEMMTensorParallelContext, persistent: bool = True,
            autotune: bool = False, straggler_option: Optional[Tuple[int, float]] = None,
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a`` [M/W, K], ``b`` [N_local, K] -> [M, N_local].

    ``straggler_option=(rank, seconds)`` delays that rank on the host before the launch (a test aid; the
    reference delays inside the kernel, allgather_gemm.py:602).  ``autotune=True`` lets the contextual autotuner time
    the whole call on all ranks for every candidate of ``AG_GEMM_TUNE_SPACE`` (push flavour, comm CTAs) the first time
    a shape is seen, and uses the winner afterwards; ``ops.tuned_configs`` holds the winners measured on B200.
    """
    rt = ctx.rt
    if autotune and rt.is_cuda and ctx.num_ranks > 1:
        return _ag_gemm_tuned(a, b, ctx, straggler_option=straggler_option, out=out)
    if straggler_option is not None and straggler_option[0] == ctx.rank:
        time.sleep(float(straggler_option[1]))
    if not _native.use_native(a, b) or a.dtype != torch.bfloat16:
        res = ag_gemm_reference(a, b, rt.group)
        if out is not None:
            out.copy_(res)
            return out
        return res
    lib = _native.load(True)
    W = ctx.num_ranks
    if W == 1:
        from .gemm import gemm
        return gemm(a, b, out=out)
    a = a.contiguous()
    if b.stride(-1) != 1:
        b = b.contiguous()
    m, K = a.shape
    N = b.shape[0]
    if K != ctx.K:
        raise ValueError(f"ag_gemm: K={K} differs from the context's K={ctx.K}")
    if out is None:
        out = torch.empty((m * W, N), dtype=a.dtype, device=a.device)
    n_sms = ctx.num_ctas or sm_count(a.device)
    pair = use_cta_pair(ctx.kernel_form, m, N, out)
    # knob precedence: a configuration the autotuner is trying / has chosen, then the context, then the table of
    # measured winners, then the model
    from .tuned_configs import lookup as tuned_lookup
    cfg = current_config()
    if cfg:                                   # the autotuner's candidate / winner overrides the context
        want_mc = cfg.get("use_multimem", ctx.use_multimem)
        want_comm = cfg.get("n_comm_ctas", ctx.n_comm_ctas)
    else:
        cfg = tuned_lookup("ag_gemm", W, m, N, K) or {}
        want_mc = ctx.use_multimem if ctx.mc_explicit else cfg.get("use_multimem", ctx.use_multimem)
        want_comm = ctx.n_comm_ctas or cfg.get("n_comm_ctas", 0)
    mc = bool(want_mc and rt.has_multicast)
    if pair and mc:
        n_comm = want_comm if want_comm in (2, 4, 8) else 4
    else:
        n_comm = want_comm or pick_comm_ctas(m, N, W, ctx.BLOCK_N, n_sms, pair, K)
        n_comm = max(1, min(n_comm, n_sms - 1))
        if pair and n_comm % 2:
            n_comm += 1
    if rt.config.debug:
        from .common import poison_unused_parity
        poison_unused_parity(ctx.workspace, ctx.calls)
    lib.ag_gemm_bf16(rt.heap, a, b, out, ctx.workspace, ctx.flags, ctx.ctx_dev, ctx.max_seg_rows, ctx.max_chunks,
                     n_comm, 512 if pair else ctx.BLOCK_N, n_sms, mc,
                     rt.config.wait_timeout_s, ctx.stats)
    ctx.calls += 1
    return out

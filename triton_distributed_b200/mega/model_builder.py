"""Builder of the decode megakernel: records operators, lets the C++ scheduler turn them into per-SM task queues, and
launches the persistent kernel.

API of the reference: ``ModelBuilder`` (python/triton_dist/mega_triton_kernel/models/model_builder.py:86-584) with the
``make_*`` surface, ``compile()``, ``run()``, ``dump_trace()`` and ``get_sm_activity()``.  The reference generates and
JIT-compiles a Triton kernel per model; here one ahead-of-time compiled task interpreter (``csrc/mega/megakernel.cu``)
executes the queues built by ``csrc/mega/scheduler.cc``.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import _native
from ..ops.common import new_ctx_dev
from ..runtime import get_runtime
from ..tools import profiler as prof_tools

T_RMSNORM, T_LINEAR, T_ROPE_KV, T_ATTN_SPLIT, T_ATTN_COMBINE, T_SILU_MUL = 1, 2, 3, 4, 5, 6
T_PREFETCH, T_BARRIER, T_ALLREDUCE = 7, 8, 9
TASK_NAMES = {1: "rms_norm", 2: "linear", 3: "qk_norm_rope_kv", 4: "flash_decode_split", 5: "flash_decode_combine",
              6: "silu_mul", 7: "prefetch_l2", 8: "barrier_all", 9: "all_reduce"}
PREFETCH_CHUNK_BYTES = 384 * 1024     # one pass of the CTA: 192 threads x 2 KB requests


def _i32(v: int) -> int:
    """The 32-bit pattern ``v`` as the signed value an int32 field holds."""
    v &= 0xFFFFFFFF
    return v - (1 << 32) if v & 0x80000000 else v


class _LoggingScheduler:
    """Wraps the native scheduler and records every call so that ``compile`` can replay it with final addresses."""

    def __init__(self, native, log):
        self._n, self._log = native, log

    def add_op(self, ptrs, ints, floats):
        idx = self._n.add_op(ptrs, ints, floats)
        self._log.append(("op", list(ptrs), list(ints), list(floats), idx))
        return idx

    def add_stage(self, ty, op, n0, n1, n2, dep):
        st = self._n.add_stage(ty, op, n0, n1, n2, dep)
        self._log.append(("stage", ty, op, n0, n1, n2, dep))
        return st

    def __getattr__(self, name):
        return getattr(self._n, name)



class ModelBuilder:
    def __init__(self, batch: int, rank: Optional[int] = None, world_size: Optional[int] = None, num_sms: Optional[int] = None,
                 policy: str = "round_robin", enable_profiling: bool = False, use_multimem: bool = True):
        self.rt = get_runtime()
        self.lib = _native.load(True)
        self.rank = self.rt.rank if rank is None else rank
        self.world_size = self.rt.world_size if world_size is None else world_size
        self.batch = int(batch)
        if not 1 <= self.batch <= 64:
            raise ValueError("the decode megakernel handles 1..64 sequences")
        self.device = self.rt.device
        self.num_sms = num_sms or torch.cuda.get_device_properties(self.device).multi_processor_count
        self.policy = 1 if policy == "zig_zag" else 0
        self.use_multimem = use_multimem and self.rt.has_multicast
        self._log: List[tuple] = []
        self.sched = _LoggingScheduler(self.lib.MegaScheduler(), self._log)
        self.mpad = self.lib.megakernel_mpad(self.batch)
        self._tmaps: List[torch.Tensor] = []
        self._tmap_index: Dict[tuple, int] = {}
        self._producer: Dict[int, int] = {}       # data_ptr -> stage that wrote it last
        self._keep: List[torch.Tensor] = []
        self._ar_ops: List[dict] = []
        self._bar_ops: List[int] = []
        self._fused_ar_stages = set()
        self._max_n = 0
        self._max_tiles = 0
        self._last_stage = -1
        self.enable_profiling = enable_profiling
        self.compiled = False

    # ------------------------------------------------------------------ helpers
    def _tmap(self, t: torch.Tensor, box_rows: int) -> int:
        key = (t.data_ptr(), tuple(t.shape), t.stride(0), box_rows)
        if key not in self._tmap_index:
            self._tmap_index[key] = len(self._tmaps)
            self._tmaps.append(self.lib.make_tensor_map(t, box_rows))
        return self._tmap_index[key]

    def _dep(self, *inputs) -> int:
        deps = [self._producer[t.data_ptr()] for t in inputs if t is not None and t.data_ptr() in self._producer]
        return max(deps) if deps else -1

    def _wrote(self, stage: int, *outs):
        for t in outs:
            if t is not None:
                self._producer[t.data_ptr()] = stage
        self._last_stage = stage

    def _ptr(self, t) -> int:
        if t is None:
            return 0
        self._keep.append(t)
        return t.data_ptr()

    # ------------------------------------------------------------------ make_* surface
    def make_rms_norm(self, x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float = 1e-6,
                      residual: Optional[torch.Tensor] = None) -> int:
        """out = rmsnorm(x (+ residual)) * weight; ``residual`` is updated in place with the sum."""
        H = x.shape[-1]
        op = self.sched.add_op([self._ptr(x), self._ptr(residual), self._ptr(weight), self._ptr(out)], [H, x.stride(0)], [eps])
        st = self.sched.add_stage(T_RMSNORM, op, self.batch, 1, 1, self._dep(x, residual))
        self._wrote(st, out, residual)
        return st

    def make_add(self, a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None):
        """Residual adds are folded into the following ``make_rms_norm(..., residual=...)``; nothing is scheduled."""
        return self._last_stage

    def make_linear(self, x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, all_reduce: bool = False,
                    splits: int = 0) -> int:
        """out [B, N] = x [B, K] @ weight [N, K]^T, optionally summed over the ranks inside the same tasks."""
        N, K = weight.shape
        tiles = (N + 127) // 128
        if splits <= 0:
            splits = int(self.lib.skinny_gemm_pick_splits(N, K, self.num_sms, self.batch))
        ar = bool(all_reduce and self.world_size > 1)
        self._max_n = max(self._max_n, N)
        self._max_tiles = max(self._max_tiles, tiles)
        ints = [N, K, splits, self._tmap(weight, 128), self._tmap(x, self.mpad), out.stride(0), 1 if ar else 0, tiles, tiles]
        op = self.sched.add_op([self._ptr(out), 0, 0], ints, [])
        if ar:
            self._ar_ops.append({"op": op, "N": N, "tiles": tiles, "out": out, "ints": ints})
        st = self.sched.add_stage(T_LINEAR, op, tiles, splits, 1, self._dep(x))
        if all_reduce:
            self._fused_ar_stages.add(st)
        self._wrote(st, out)
        return st

    make_qkv_proj = make_o_proj = make_fc1 = make_fc2 = make_linear

    def make_lm_head(self, x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> int:
        """Logits of the local vocabulary shard: a linear stage without all-reduce."""
        return self.make_linear(x, weight, out, all_reduce=False)

    def make_allreduce(self, x: torch.Tensor, out: Optional[torch.Tensor] = None, chunk_cols: int = 1024) -> int:
        """Sum ``x`` [B, N] over the ranks.  A tensor produced by ``make_linear(..., all_reduce=True)`` is already
        summed (the all-reduce ran inside those tasks): nothing is scheduled for it.  Otherwise stand-alone all-reduce
        tasks, one per ``chunk_cols`` columns, write ``out`` (default: in place).  All-reduces alternate between two
        staging buffers: between two of them that share a buffer (every second one, and the same one of the next launch)
        there must be another all-reduce or a ``make_barrier_all_intra_node``, as in the reference's barrier + all-reduce
        pairs, so that no rank overwrites a buffer a slower rank is still summing."""
        st = self._producer.get(x.data_ptr(), -1)
        if st >= 0 and st in self._fused_ar_stages:
            return st
        out = x if out is None else out
        N = x.shape[-1]
        if N % 8 or chunk_cols % 8:
            raise ValueError("make_allreduce: N and chunk_cols must be multiples of 8")
        chunks = (N + chunk_cols - 1) // chunk_cols
        self._max_tiles = max(self._max_tiles, chunks)
        ints = [N, x.stride(0), out.stride(0), chunk_cols, chunks]
        op = self.sched.add_op([self._ptr(x), 0, 0, self._ptr(out)], ints, [])
        if self.world_size > 1:
            self._ar_ops.append({"op": op, "N": N, "tiles": chunks, "out": out, "ints": ints, "standalone": True})
        stage = self.sched.add_stage(T_ALLREDUCE, op, chunks, 1, 1, self._dep(x))
        self._wrote(stage, out)
        return stage

    def make_barrier_all_intra_node(self) -> int:
        """One task that holds its SM until every rank has reached it (epoch flags in the heap, nothing to reset).  Stages
        scheduled after it depend on it only if they are given its stage through a tensor written by it; the reference
        uses it around its all-reduce task (model_builder.py:467-486), which the flag protocol here does not need."""
        op = self.sched.add_op([0], [], [])
        self._bar_ops.append(op)
        stage = self.sched.add_stage(T_BARRIER, op, 1, 1, 1, self._last_stage)
        self._last_stage = stage
        return stage

    def make_prefetch(self, weight: torch.Tensor, after: Optional[torch.Tensor] = None) -> int:
        """Request ``weight`` into L2 ahead of the operator that will stream it (cp.async.bulk.prefetch.L2, asynchronous).
        ``after``: a tensor whose producing stage must be complete before the requests are issued (so that they do not
        compete with the operator that is running now); None = as soon as an SM reaches the task."""
        total = weight.numel() * weight.element_size()
        if not weight.is_contiguous() or weight.data_ptr() % 16:
            raise ValueError("make_prefetch: contiguous, 16-byte aligned tensor expected")
        chunks = max(1, (total + PREFETCH_CHUNK_BYTES - 1) // PREFETCH_CHUNK_BYTES)
        op = self.sched.add_op([self._ptr(weight)], [_i32(total & 0xFFFFFFFF), _i32(total >> 32), PREFETCH_CHUNK_BYTES], [])
        return self.sched.add_stage(T_PREFETCH, op, chunks, 1, 1, self._dep(after) if after is not None else -1)

    def make_qk_norm_rope_update_kvcache(self, qkv: torch.Tensor, q_norm_w, k_norm_w, q_out: torch.Tensor,
                                         k_cache: torch.Tensor, v_cache: torch.Tensor, kv_offset: torch.Tensor,
                                         num_q_heads: int, num_kv_heads: int, head_dim: int, eps: float = 1e-6,
                                         rope_theta: float = 1e6) -> int:
        """k_cache / v_cache: one layer of a dense cache [B, max_len, Hkv, D]; ``kv_offset`` int32 [B] = position of the
        token being decoded."""
        import math
        max_len = k_cache.shape[1]
        op = self.sched.add_op([self._ptr(qkv), self._ptr(q_norm_w), self._ptr(k_norm_w), self._ptr(q_out), self._ptr(k_cache),
                                self._ptr(v_cache), self._ptr(kv_offset)],
                               [num_q_heads, num_kv_heads, head_dim, qkv.stride(0), max_len], [eps, math.log2(rope_theta)])
        st = self.sched.add_stage(T_ROPE_KV, op, self.batch, 1, 1, self._dep(qkv))
        self._wrote(st, q_out, k_cache, v_cache)
        return st

    def make_flash_decode(self, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, kv_lens: torch.Tensor,
                          out: torch.Tensor, num_q_heads: int, num_kv_heads: int, head_dim: int, scale: Optional[float] = None,
                          splits: int = 0) -> int:
        """Split-KV decode attention over a dense cache [B, max_len, Hkv, D]; ``kv_lens`` int32 [B] includes the new token."""
        from ..ops.attention import pick_kv_splits
        max_len = k_cache.shape[1]
        group = num_q_heads // num_kv_heads
        chunks = (group + 15) // 16
        if splits <= 0:
            # tasks of one SM run one after the other, so there is no point in more split tasks than SMs
            blocks = max(1, (max_len + 63) // 64)
            splits = max(1, min(blocks, 64, self.num_sms // max(1, self.batch * num_kv_heads * chunks)))
        ws = torch.empty(self.batch * num_q_heads * splits * (head_dim + 1), dtype=torch.float32, device=self.device)
        bt = torch.arange(self.batch, dtype=torch.int32, device=self.device).contiguous()
        scale = scale if scale is not None else head_dim ** -0.5
        op = self.sched.add_op([self._ptr(q), self._ptr(ws), self._ptr(k_cache), self._ptr(v_cache), self._ptr(kv_lens),
                                self._ptr(bt), self._ptr(out)], [num_q_heads, num_kv_heads, head_dim, splits, max_len, 1],
                               [scale])
        s1 = self.sched.add_stage(T_ATTN_SPLIT, op, self.batch, splits, num_kv_heads * chunks, self._dep(q, k_cache, v_cache))
        s2 = self.sched.add_stage(T_ATTN_COMBINE, op, self.batch, num_q_heads, 1, s1)   # one task per (sequence, head)
        self._wrote(s2, out)
        return s2

    # ------------------------------------------------------------------ prefill tasks of the reference
    def _prefill_not_built(self, name: str):
        raise NotImplementedError(
            f"ModelBuilder.{name}: the task interpreter of this package is decode-only (one token per sequence and "
            "step).  Prefill runs through the layer path (models.DenseLLM.inference with ops.flash_attn_varlen, the "
            "tcgen05 prefill kernel); the megakernel takes over from the first decode step "
            "(reference: mega_triton_kernel/models/model_builder.py make_flash_attn / make_qkv_pack_*).")

    def make_flash_attn(self, *args, **kwargs):
        self._prefill_not_built("make_flash_attn")

    def make_qkv_pack_flash_attn(self, *args, **kwargs):
        self._prefill_not_built("make_qkv_pack_flash_attn")

    def make_qkv_pack_qk_norm_rope_split_v(self, *args, **kwargs):
        self._prefill_not_built("make_qkv_pack_qk_norm_rope_split_v")

    def make_silu_mul_up(self, x: torch.Tensor, out: torch.Tensor) -> int:
        I = x.shape[-1] // 2
        nchunks = max(1, min(16, self.num_sms // max(1, self.batch), I // 2048))
        op = self.sched.add_op([self._ptr(x), self._ptr(out)], [I, x.stride(0), nchunks], [])
        st = self.sched.add_stage(T_SILU_MUL, op, self.batch, nchunks, 1, self._dep(x))
        self._wrote(st, out)
        return st

    # ------------------------------------------------------------------ compile / run
    def compile(self):
        rt, dev = self.rt, self.device
        # cross-rank buffers of the fused all-reduces: two ping-pong partial buffers + per-op flags
        if self._ar_ops:
            n_max = max(o["N"] for o in self._ar_ops)
            slots = 1 if self.use_multimem else self.world_size
            self.partial = rt.symm_tensor((2, slots, self.batch, n_max), torch.bfloat16, zero=False)
            self.ar_flags = rt.symm_tensor((len(self._ar_ops), self.world_size, self._max_tiles), torch.int32)
            # the op records were added before the buffers existed: rebuild the scheduler's op table entries
            # (pointers 1 and 2 of every all-reduce op) through a second scheduler with identical stages
        if self._bar_ops:
            self.bar_flags = rt.symm_tensor((len(self._bar_ops), max(self.world_size, 8)), torch.int32)
        sched2 = self.lib.MegaScheduler()
        self._rebuild(sched2)
        self.sched = sched2
        self.sched.schedule(self.num_sms, self.policy)
        self.tasks = self.sched.tasks_tensor().to(dev)
        self.offsets = self.sched.offsets_tensor().to(dev)
        self.ops_dev = self.sched.ops_tensor().to(dev)
        tm = torch.stack(self._tmaps) if self._tmaps else torch.zeros((1, 128), dtype=torch.uint8)
        self.tmaps_dev = tm.to(dev).contiguous()
        self.scoreboard = torch.zeros(max(self.sched.scoreboard_size, 1), dtype=torch.int32, device=dev)
        self.acc = torch.zeros(self.batch * max(self._max_n, 1), dtype=torch.float32, device=dev)
        self.counters = torch.zeros(max(self._max_tiles, 1), dtype=torch.int32, device=dev)
        self.ctx_dev = new_ctx_dev(rt)
        self.profile_buf = prof_tools.create_buffer(1 << 18, dev) if self.enable_profiling else None
        torch.cuda.synchronize()
        rt.host_barrier()
        self.compiled = True

    def _rebuild(self, sched2):
        """Re-emit ops and stages into a fresh scheduler, now with the all-reduce buffers' addresses."""
        ar_index = {o["op"]: i for i, o in enumerate(self._ar_ops) if self.world_size > 1}
        self._replay_ops(sched2, ar_index)

    # ops / stages are recorded twice: once while building (to learn sizes) and once here with final pointers.  To keep
    # that simple the builder logs every call and replays the log.
    def _replay_ops(self, sched2, ar_index):
        for rec in self._log:
            kind = rec[0]
            if kind == "op":
                _, ptrs, ints, floats, idx = rec
                if idx in ar_index:
                    i = ar_index[idx]
                    buf = self.partial[i & 1]
                    ptrs = [ptrs[0], buf.data_ptr(), self.ar_flags[i].data_ptr()] + list(ptrs[3:])
                elif idx in self._bar_ops:
                    ptrs = [self.bar_flags[self._bar_ops.index(idx)].data_ptr()]
                sched2.add_op(ptrs, ints, floats)
            else:
                _, ty, op, n0, n1, n2, dep = rec
                sched2.add_stage(ty, op, n0, n1, n2, dep)

    def run(self):
        if not self.compiled:
            raise RuntimeError("call compile() first")
        self.lib.mega_launch(self.rt.heap, self.tasks, self.offsets, self.ops_dev, self.tmaps_dev, self.scoreboard, self.acc,
                             self.counters, self.ctx_dev, self.batch, self.num_sms, bool(self.use_multimem), self.profile_buf,
                             self.rt.config.wait_timeout_s)

    # ------------------------------------------------------------------ introspection
    def tasks_per_sm(self):
        return self.sched.tasks_per_sm()

    def dump_trace(self, path: str):
        if self.profile_buf is None:
            raise RuntimeError("build with enable_profiling=True")
        torch.cuda.synchronize()
        return prof_tools.to_chrome_trace(prof_tools.decode(self.profile_buf), TASK_NAMES, path)

    def get_sm_activity(self):
        if self.profile_buf is None:
            raise RuntimeError("build with enable_profiling=True")
        torch.cuda.synchronize()
        return prof_tools.sm_activity(prof_tools.decode(self.profile_buf))

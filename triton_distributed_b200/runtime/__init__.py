"""Process bootstrap, symmetric heap, host-side synchronisation and bounded-wait error reporting.

Covers what the reference does in ``python/triton_dist/utils.py``: ``initialize_distributed`` (:182-205),
``finalize_distributed`` (:145-148), ``nvshmem_create_tensor(s)`` (:114-136), ``nvshmem_free_tensor_sync``
(:139-142), ``nvshmem_barrier_all_on_stream`` (:162-164) — with the NVSHMEM heap replaced by the native
cuMem/NVLS heap of this package (``csrc/symm_heap.cc``) and every device wait bounded.

One process per GPU.  ``torch.distributed`` (NCCL + gloo) is only the bootstrap side channel and the
baseline; on a machine without a GPU the runtime still comes up (gloo only, ordinary CPU tensors stand
in for symmetric tensors) so the torch reference backend of every op can be tested.
"""
from __future__ import annotations

import atexit
import datetime
import os
import random
import threading
import uuid
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch
import torch.distributed as dist

from .. import _native

__all__ = [
    "DistConfig", "CommTimeoutError", "Runtime", "initialize_distributed", "finalize_distributed", "get_runtime",
    "symm_tensor", "symm_tensors", "symm_free", "nvshmem_create_tensor", "nvshmem_create_tensors",
    "nvshmem_free_tensor_sync", "nvshmem_barrier_all_on_stream", "barrier_all_on_stream", "STATUS_CODES",
    "KERNEL_NAMES", "Watchdog",
]

STATUS_CODES = {0: "ok", 1: "timeout waiting for a flag", 2: "timeout waiting for an mbarrier",
                3: "timeout in a barrier", 4: "bad argument", 5: "aborted"}
KERNEL_NAMES = {0: "none", 1: "gemm", 2: "ag_gemm", 3: "gemm_rs", 4: "gemm_ar", 5: "all_reduce", 6: "all_gather",
                7: "reduce_scatter", 8: "barrier", 9: "all_to_all", 10: "ep_dispatch", 11: "ep_combine",
                12: "flash_decode", 13: "megakernel", 14: "group_gemm", 15: "moe_reduce", 16: "p2p",
                17: "primitive", 18: "gemv"}


class CommTimeoutError(RuntimeError):
    """A bounded device-side wait gave up; ``record`` holds the kernel's report."""

    def __init__(self, record: dict):
        self.record = dict(record)
        super().__init__(
            "device wait gave up: {} in kernel '{}' (site {}, block {}, peer {}, index {}, expected {}, observed {})".format(
                STATUS_CODES.get(record.get("code"), record.get("code")),
                KERNEL_NAMES.get(record.get("kernel"), record.get("kernel")), record.get("where"),
                record.get("block"), record.get("peer"), record.get("index"), record.get("expected"),
                record.get("observed")))


def _env_int(name: str, default: int) -> int:
    v = os.environ.get(name)
    return int(float(v)) if v not in (None, "") else default


def _env_float(name: str, default: float) -> float:
    v = os.environ.get(name)
    return float(v) if v not in (None, "") else default


@dataclass
class DistConfig:
    """Run-time switches; every field can be set through an environment variable ``TDB200_*``.

    The reference spreads the same knobs over NVSHMEM environment variables
    (``NVSHMEM_SYMMETRIC_SIZE``, ``NVSHMEM_DISABLE_CUDA_VMM`` in scripts/launch.sh:128-139).
    """
    heap_bytes: int = field(default_factory=lambda: _env_int("TDB200_SYMM_HEAP_BYTES", 4 << 30))
    nvls: bool = field(default_factory=lambda: _env_int("TDB200_NVLS", 1) != 0)
    heap_mode: str = field(default_factory=lambda: os.environ.get("TDB200_HEAP_MODE", "vmm"))
    wait_timeout_s: float = field(default_factory=lambda: _env_float("TDB200_WAIT_TIMEOUT_S", 10.0))
    debug: bool = field(default_factory=lambda: _env_int("TDB200_DEBUG", 0) != 0)
    pg_timeout_s: float = field(default_factory=lambda: _env_float("TDB200_PG_TIMEOUT_S", 1800.0))


class Runtime:
    """Per-process state: ranks, process groups, the symmetric heap and its status page."""

    def __init__(self, config: DistConfig):
        self.config = config
        self.rank = 0
        self.world_size = 1
        self.local_rank = 0
        self.local_world_size = 1
        self.device = torch.device("cpu")
        self.group: Optional[dist.ProcessGroup] = None       # accelerator group (NCCL on GPU, gloo on CPU)
        self.cpu_group: Optional[dist.ProcessGroup] = None   # gloo side channel
        self.heap = None                                     # native SymmHeap, None on CPU
        self._allocs = {}                                    # data_ptr -> (offset, nbytes)
        self._barrier_flags = None
        self._barrier_ctx = None
        self._own_pg = False
        self._lock = threading.Lock()

    # ------------------------------------------------------------------ properties
    @property
    def is_cuda(self) -> bool:
        return self.device.type == "cuda"

    @property
    def has_multicast(self) -> bool:
        return self.heap is not None and bool(self.heap.has_multicast)

    # ------------------------------------------------------------------ heap
    def _init_heap(self):
        lib = _native.load(True)
        cfg = self.config
        session = [uuid.uuid4().hex[:16] if self.rank == 0 else None]
        if self.world_size > 1:
            dist.broadcast_object_list(session, src=0, group=self.cpu_group)
        want_mc = cfg.nvls and self.world_size > 1
        self.heap = lib.SymmHeap(self.rank, self.world_size, self.device.index, int(cfg.heap_bytes), session[0], want_mc)
        if cfg.heap_mode == "ipc" and self.world_size > 1:
            self.heap.create_ipc()
            handles = [None] * self.world_size
            dist.all_gather_object(handles, self.heap.ipc_handle(), group=self.cpu_group)
            self.heap.map_ipc(handles)
            dist.barrier(group=self.cpu_group)
        else:
            self.heap.create()
            if self.world_size > 1:
                dist.barrier(group=self.cpu_group)
                self.heap.exchange_and_map()
                dist.barrier(group=self.cpu_group)
                ok = [True]
                try:
                    self.heap.multicast_setup()
                except RuntimeError as e:  # no NVLS on this machine: peer-to-peer algorithms only
                    ok = [False]
                    self._mc_error = str(e)
                oks = [None] * self.world_size
                dist.all_gather_object(oks, ok[0], group=self.cpu_group)
                if all(oks) and want_mc:
                    self.heap.multicast_bind()
                dist.barrier(group=self.cpu_group)
        # barrier state lives in the heap itself
        self._barrier_flags = self.symm_tensor((64,), torch.int32)
        self._barrier_ctx = torch.zeros(8, dtype=torch.int32, device=self.device)
        self._barrier_ctx[0] = 1
        torch.cuda.synchronize()
        if self.world_size > 1:
            dist.barrier(group=self.cpu_group)

    def symm_tensor(self, shape: Sequence[int], dtype: torch.dtype, zero: bool = True, sync: bool = True) -> torch.Tensor:
        """Allocate a tensor at the same heap offset on every rank (collective: same call order on all ranks).

        Like the reference's ``nvshmem_create_tensor`` the call ends with a barrier over all ranks (``sync``): when
        it returns, every rank has allocated AND zero-filled its copy, so a peer may write into it or raise a flag in
        it right away.  Callers that allocate several tensors in a row may pass ``sync=False`` and finish with
        ``torch.cuda.synchronize(); host_barrier()`` themselves."""
        shape = tuple(int(s) for s in shape)
        if self.heap is None:
            return torch.zeros(shape, dtype=dtype, device=self.device)
        nbytes = int(np.prod(shape, dtype=np.int64)) * torch.empty((), dtype=dtype).element_size()
        off = self.heap.alloc(max(nbytes, 16), 256)
        t = self.heap.tensor(off, list(shape), dtype)
        self._allocs[t.data_ptr()] = (off, nbytes)
        if zero:
            t.zero_()
        if sync and self.world_size > 1:
            torch.cuda.synchronize()
            self.host_barrier()
        return t

    def symm_tensors(self, shape: Sequence[int], dtype: torch.dtype) -> List[torch.Tensor]:
        """Allocate and return the views of the allocation on every rank (index = rank)."""
        t = self.symm_tensor(shape, dtype)
        return [t if r == self.rank else self.peer_view(t, r) for r in range(self.world_size)]

    def offset_of(self, t: torch.Tensor) -> int:
        return int(self.heap.offset_of(t))

    def peer_view(self, t: torch.Tensor, peer: int) -> torch.Tensor:
        """The same heap object as seen on ``peer`` (a P2P-mapped tensor)."""
        if self.heap is None:
            raise RuntimeError("peer views need the GPU heap")
        v = self.heap.tensor(self.offset_of(t), list(t.shape), t.dtype, peer=peer)
        return v

    def multicast_view(self, t: torch.Tensor) -> torch.Tensor:
        return self.heap.tensor(self.offset_of(t), list(t.shape), t.dtype, multicast=True)

    def symm_free(self, t: torch.Tensor):
        if self.heap is None:
            return
        ent = self._allocs.pop(t.data_ptr(), None)
        if ent is not None:
            self.heap.free(ent[0])

    def is_symmetric(self, t: torch.Tensor) -> bool:
        if self.heap is None or not t.is_cuda:
            return False
        p = t.data_ptr()
        return self.heap.local_base <= p < self.heap.local_base + self.heap.heap_bytes

    # ------------------------------------------------------------------ sync
    def barrier_all_on_stream(self, stream: Optional[torch.cuda.Stream] = None):
        """Rank barrier enqueued on a CUDA stream (a one-CTA kernel over heap flags); gloo barrier on CPU."""
        if self.heap is None:
            if self.world_size > 1:
                dist.barrier(group=self.cpu_group)
            return
        lib = _native.load(True)
        if stream is None:
            lib.barrier_all(self.heap, self._barrier_flags, self._barrier_ctx, self.config.wait_timeout_s)
        else:
            with torch.cuda.stream(stream):
                lib.barrier_all(self.heap, self._barrier_flags, self._barrier_ctx, self.config.wait_timeout_s)

    def host_barrier(self):
        if self.world_size > 1:
            dist.barrier(group=self.cpu_group)

    # ------------------------------------------------------------------ status
    def read_status(self) -> dict:
        return dict(self.heap.read_status()) if self.heap is not None else {"code": 0}

    def check_status(self, sync: bool = True):
        """Raise :class:`CommTimeoutError` if a kernel reported a wait that gave up."""
        if self.heap is None:
            return
        if sync:
            torch.cuda.synchronize()
        rec = self.read_status()
        if rec.get("code", 0) != 0:
            self.heap.clear_status()
            raise CommTimeoutError(rec)

    def abort(self):
        """Make every spinning kernel of this rank give up (they poll the abort word)."""
        if self.heap is not None:
            self.heap.set_abort(1)

    def clear_abort(self):
        if self.heap is not None:
            self.heap.set_abort(0)
            self.heap.clear_status()

    # ------------------------------------------------------------------ teardown
    def finalize(self):
        if self.heap is not None:
            try:
                torch.cuda.synchronize()
                if self.world_size > 1 and dist.is_initialized():
                    dist.barrier(group=self.cpu_group)
            except Exception:
                pass
            self._barrier_flags = None
            self.heap.destroy()
            self.heap = None
        # On a GPU the process group is left to torch's own exit handling: destroying it here can block when CUDA graphs
        # that captured NCCL work are still alive in the caller.  CPU ranks (gloo) destroy it: a gloo group that is
        # still alive at interpreter exit can abort the process from its background threads
        # ("terminate called without an active exception").
        if not self.is_cuda and self._own_pg and dist.is_initialized():
            try:
                dist.barrier()
                dist.destroy_process_group()
            except Exception:
                pass


class Watchdog:
    """Host thread that polls the status page and an epoch counter.

    Calls ``on_error(record)`` as soon as a kernel reports a failed wait, without waiting for a
    stream synchronisation (the page is pinned host memory written by the GPU).
    """

    def __init__(self, runtime: Runtime, on_error=None, period_s: float = 0.05):
        self.runtime = runtime
        self.on_error = on_error
        self.period_s = period_s
        self.last_record: Optional[dict] = None
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def start(self):
        self._thread.start()
        return self

    def stop(self):
        self._stop.set()
        self._thread.join(timeout=2.0)

    def _run(self):
        while not self._stop.wait(self.period_s):
            if self.runtime.heap is None:
                continue
            rec = self.runtime.read_status()
            if rec.get("code", 0) != 0:
                self.last_record = rec
                if self.on_error is not None:
                    self.on_error(rec)
                return


_RUNTIME: Optional[Runtime] = None


def get_runtime() -> Runtime:
    if _RUNTIME is None:
        raise RuntimeError("call initialize_distributed() first")
    return _RUNTIME


def _init_seed(seed: int):
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
    np.random.seed(seed % (2 ** 32))
    random.seed(seed)


def initialize_distributed(seed: Optional[int] = None, config: Optional[DistConfig] = None,
                           device: Optional[str] = None, with_heap: bool = True):
    """Bring up the process group(s) and the symmetric heap; returns the tensor-parallel process group.

    Reads ``RANK`` / ``LOCAL_RANK`` / ``WORLD_SIZE`` / ``MASTER_ADDR`` / ``MASTER_PORT`` as set by torchrun; without
    them a single-rank runtime is created.  ``device="cpu"`` forces the gloo-only runtime.
    """
    global _RUNTIME
    if _RUNTIME is not None:
        return _RUNTIME.group
    rt = Runtime(config or DistConfig())
    rt.rank = int(os.environ.get("RANK", 0))
    rt.world_size = int(os.environ.get("WORLD_SIZE", 1))
    rt.local_rank = int(os.environ.get("LOCAL_RANK", rt.rank))
    rt.local_world_size = int(os.environ.get("LOCAL_WORLD_SIZE", rt.world_size))
    use_cuda = torch.cuda.is_available() and device != "cpu"
    if use_cuda:
        torch.cuda.set_device(rt.local_rank)
        rt.device = torch.device("cuda", rt.local_rank)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if "MASTER_PORT" not in os.environ:
            import socket
            with socket.socket() as s:
                s.bind(("127.0.0.1", 0))
                os.environ["MASTER_PORT"] = str(s.getsockname()[1])
        backend = "cpu:gloo,cuda:nccl" if (use_cuda and rt.world_size > 1) else "gloo"
        dist.init_process_group(backend=backend, rank=rt.rank, world_size=rt.world_size,
                                timeout=datetime.timedelta(seconds=rt.config.pg_timeout_s))
        rt._own_pg = True
    ranks = list(range(rt.world_size))
    rt.group = dist.new_group(ranks=ranks, backend="nccl" if (use_cuda and rt.world_size > 1) else "gloo")
    rt.cpu_group = dist.new_group(ranks=ranks, backend="gloo")
    _init_seed((seed if seed is not None else 0) + rt.rank)
    _RUNTIME = rt
    if use_cuda and with_heap:
        rt._init_heap()
    atexit.register(_atexit_finalize)
    return rt.group


def _atexit_finalize():
    global _RUNTIME
    if _RUNTIME is not None and _RUNTIME.heap is not None:
        try:
            torch.cuda.synchronize()
            _RUNTIME.heap.destroy()
        except Exception:
            pass
        _RUNTIME.heap = None


def finalize_distributed():
    global _RUNTIME
    if _RUNTIME is not None:
        _RUNTIME.finalize()
        _RUNTIME = None


def symm_tensor(shape, dtype) -> torch.Tensor:
    return get_runtime().symm_tensor(shape, dtype)


def symm_tensors(shape, dtype) -> List[torch.Tensor]:
    return get_runtime().symm_tensors(shape, dtype)


def symm_free(t: torch.Tensor):
    get_runtime().symm_free(t)


# Names kept from the reference API (python/triton_dist/utils.py:114-164).
def nvshmem_create_tensor(shape, dtype) -> torch.Tensor:
    return symm_tensor(shape, dtype)


def nvshmem_create_tensors(shape, dtype, rank=None, local_world_size=None) -> List[torch.Tensor]:
    return symm_tensors(shape, dtype)


def nvshmem_free_tensor_sync(t: torch.Tensor):
    rt = get_runtime()
    if rt.is_cuda:
        torch.cuda.synchronize()
    rt.host_barrier()
    rt.symm_free(t)


def barrier_all_on_stream(stream=None):
    get_runtime().barrier_all_on_stream(stream)


def nvshmem_barrier_all_on_stream(stream=None):
    get_runtime().barrier_all_on_stream(stream)

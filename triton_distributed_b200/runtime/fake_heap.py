"""A symmetric heap made of POSIX shared memory, for running the library's flag protocols among CPU ranks.

On a GPU box every rank maps every rank's heap (``cuMemMap`` of exported handles) and kernels exchange data with plain
stores to ``peer_base[r] + offset`` and signals with release stores to epoch flags.  This module gives CPU processes the
same shape: one shared-memory segment per rank, the same offset arithmetic, ``signal`` / ``wait_until`` with a time limit
and a status record instead of an endless spin.  The protocols below (:func:`ag_push_protocol`,
:func:`rs_scatter_protocol`) are the host restatement of what the fused kernels do: double-buffered workspaces selected
by the epoch's parity, flags that hold the epoch of the call that wrote them, nothing reset and no barrier between
calls.  They let the indexing of workspaces and flags, the "no reset" argument and the behaviour under a straggler or a
missing rank be tested without a GPU.

The reference has no counterpart: its protocols run on NVSHMEM symmetric memory only
(python/triton_dist/utils.py:90-137 ``nvshmem_create_tensor``; python/triton_dist/kernels/nvidia/allgather.py:77-191 for the push
all-gather; python/triton_dist/kernels/nvidia/gemm_reduce_scatter.py:238-330 for the scatter + reduce).
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from multiprocessing import shared_memory
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

_ALIGN = 256


class FakeWaitTimeout(RuntimeError):
    """A bounded wait on the fake heap gave up; ``record`` mirrors the device status record."""

    def __init__(self, record: Dict):
        self.record = dict(record)
        super().__init__(f"fake heap wait gave up: {record}")


class FakeSymmHeap:
    """``world`` shared-memory segments of ``nbytes`` each; rank ``rank`` owns segment ``rank``.

    Construction is collective: every rank creates its own segment, then ``barrier()`` (a callable supplied by the
    caller, e.g. a gloo barrier) separates creation from attaching to the peers' segments.  Allocation is a bump
    pointer that every rank advances identically, which is what makes offsets symmetric.
    """

    def __init__(self, name: str, rank: int, world: int, nbytes: int, barrier: Callable[[], None]):
        self.name, self.rank, self.world, self.nbytes = name, rank, world, int(nbytes)
        self._barrier = barrier
        self._own = shared_memory.SharedMemory(name=f"{name}_{rank}", create=True, size=self.nbytes)
        np.frombuffer(self._own.buf, dtype=np.uint8)[:] = 0
        barrier()
        self._segs: List[shared_memory.SharedMemory] = []
        for r in range(world):
            self._segs.append(self._own if r == rank else shared_memory.SharedMemory(name=f"{name}_{r}"))
        self._top = 0
        self._views: List[torch.Tensor] = []

    # ------------------------------------------------------------------ allocation / translation
    def tensor(self, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        """Symmetric allocation (collective: same sequence of calls on every rank).  Returns this rank's view."""
        n = int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        off = (self._top + _ALIGN - 1) // _ALIGN * _ALIGN
        if off + n > self.nbytes:
            raise MemoryError(f"fake heap exhausted: {off + n} > {self.nbytes}")
        self._top = off + n
        t = self._view(self.rank, off, shape, dtype)
        t._fake_off = off            # type: ignore[attr-defined]
        return t

    def _view(self, r: int, off: int, shape, dtype) -> torch.Tensor:
        n = int(np.prod(shape))
        t = torch.frombuffer(self._segs[r].buf, dtype=dtype, count=n, offset=off).view(*shape)
        self._views.append(t)
        return t

    def symm_at(self, t: torch.Tensor, peer: int) -> torch.Tensor:
        """The same object in ``peer``'s segment (the device ``symm_at``): bounds and rank are always checked here."""
        off = getattr(t, "_fake_off", None)
        if off is None:
            raise ValueError("symm_at: not a tensor of this heap")
        if not 0 <= peer < self.world:
            raise ValueError(f"symm_at: peer {peer} outside [0, {self.world})")
        v = self._view(peer, off, tuple(t.shape), t.dtype)
        v._fake_off = off            # type: ignore[attr-defined]
        return v

    # ------------------------------------------------------------------ signals
    @staticmethod
    def signal(flag: torch.Tensor, index: int, value: int, add: bool = False):
        """Set / add a 32-bit flag word.  Call after the data stores it publishes (x86 stores are not reordered with
        one another, the role ``st.release.sys`` plays on the device)."""
        f = flag.view(-1)
        if add:
            f[index] += value
        else:
            f[index] = value

    @staticmethod
    def wait_until(flag: torch.Tensor, index: int, expected: int, geq: bool = True, timeout_s: float = 5.0,
                   where: int = 0, peer: int = -1, abort: Optional[Callable[[], bool]] = None) -> None:
        """Poll until the flag reaches ``expected``; after ``timeout_s`` raise :class:`FakeWaitTimeout` with a record of the
        same fields as the device status page (code 1 = flag timeout, 5 = aborted)."""
        f = flag.view(-1)
        t0 = time.perf_counter()
        while True:
            v = int(f[index])
            if (v >= expected) if geq else (v == expected):
                return
            if abort is not None and abort():
                raise FakeWaitTimeout({"code": 5, "where": where, "peer": peer, "index": index, "expected": expected,
                                       "observed": v})
            if time.perf_counter() - t0 > timeout_s:
                raise FakeWaitTimeout({"code": 1, "where": where, "peer": peer, "index": index, "expected": expected,
                                       "observed": v})
            time.sleep(0)

    # ------------------------------------------------------------------ teardown
    def close(self):
        """Collective: every rank detaches, then each rank unlinks its own segment."""
        self._views.clear()
        self._barrier()
        for r, s in enumerate(self._segs):
            if r != self.rank:
                try:
                    s.close()
                except BufferError:
                    pass
        self._barrier()
        try:
            self._own.close()
        except BufferError:
            pass
        self._own.unlink()


# ---------------------------------------------------------------------------------------------------------------------
# Protocols (host restatements of the fused kernels' communication halves)
# ---------------------------------------------------------------------------------------------------------------------
@dataclass
class AgPushState:
    """Context of the push all-gather: workspace ``[2][W * rows][cols]``, flags ``[2][W][chunks]``, call count."""
    heap: FakeSymmHeap
    workspace: torch.Tensor
    flags: torch.Tensor
    rows: int
    chunk_rows: int
    calls: int = 0


def create_ag_push_state(heap: FakeSymmHeap, rows: int, cols: int, chunk_rows: int, dtype=torch.float32) -> AgPushState:
    chunks = (rows + chunk_rows - 1) // chunk_rows
    ws = heap.tensor((2, heap.world * rows, cols), dtype)
    fl = heap.tensor((2, heap.world, chunks), torch.int32)
    return AgPushState(heap, ws, fl, rows, chunk_rows)


def ag_push_protocol(st: AgPushState, shard: torch.Tensor, consume: Optional[Callable[[int, int, torch.Tensor], None]] = None,
                     timeout_s: float = 5.0, delay_s: float = 0.0) -> torch.Tensor:
    """One call of the push all-gather as the AG -> GEMM kernel's comm CTAs and producer warps run it.

    Push: for every 128-row chunk of the local shard and every peer, store the chunk into the peer's
    ``workspace[parity][rank * rows + chunk]`` and then the call epoch into the peer's ``flags[parity][rank][chunk]``.
    Consume: walk the segments starting with the local one, wait for ``flags[parity][seg][chunk] >= epoch`` and hand the
    chunk to ``consume(seg, chunk, rows)``.  ``delay_s`` makes this rank a straggler before it pushes.
    Returns the gathered ``[W * rows, cols]`` view of this call's parity buffer."""
    h = st.heap
    W, rank = h.world, h.rank
    epoch = st.calls + 1
    par = epoch & 1
    if shard.shape[0] != st.rows:
        raise ValueError("ag_push_protocol: shard rows differ from the context's")
    if delay_s > 0:
        time.sleep(delay_s)
    chunks = st.flags.shape[2]
    peers_ws = [h.symm_at(st.workspace, p) for p in range(W)]
    peers_fl = [h.symm_at(st.flags, p) for p in range(W)]
    for c in range(chunks):
        r0, r1 = c * st.chunk_rows, min((c + 1) * st.chunk_rows, st.rows)
        for d in range(W):
            p = (rank + d) % W
            peers_ws[p][par, rank * st.rows + r0: rank * st.rows + r1] = shard[r0:r1]
            FakeSymmHeap.signal(peers_fl[p][par, rank], c, epoch)
    for d in range(W):
        seg = (rank + d) % W
        for c in range(chunks):
            FakeSymmHeap.wait_until(st.flags[par, seg], c, epoch, geq=True, timeout_s=timeout_s, where=1, peer=seg)
            if consume is not None:
                r0, r1 = c * st.chunk_rows, min((c + 1) * st.chunk_rows, st.rows)
                consume(seg, c, st.workspace[par, seg * st.rows + r0: seg * st.rows + r1])
    st.calls += 1
    return st.workspace[par]


@dataclass
class RsScatterState:
    """Context of the scatter + reduce: slots ``[2][W][rows][cols]`` (one slot per source rank), flags ``[2][W][tiles]``."""
    heap: FakeSymmHeap
    slots: torch.Tensor
    flags: torch.Tensor
    rows: int
    tile_rows: int
    calls: int = 0


def create_rs_scatter_state(heap: FakeSymmHeap, rows: int, cols: int, tile_rows: int, dtype=torch.float32) -> RsScatterState:
    tiles = (rows + tile_rows - 1) // tile_rows
    sl = heap.tensor((2, heap.world, rows, cols), dtype)
    fl = heap.tensor((2, heap.world, tiles), torch.int32)
    return RsScatterState(heap, sl, fl, rows, tile_rows)


def rs_scatter_protocol(st: RsScatterState, partial: torch.Tensor, timeout_s: float = 5.0) -> torch.Tensor:
    """One call of GEMM -> reduce-scatter's communication: ``partial`` is this rank's ``[W * rows, cols]`` partial product.

    Tiles of a peer's segment go into that peer's ``slots[parity][rank]`` followed by the epoch in its
    ``flags[parity][rank][tile]``; the owner adds the tiles of its own segment as they arrive (its own partial never
    leaves the rank).  Segments are visited starting after the local one so that every rank's tiles are ready early."""
    h = st.heap
    W, rank = h.world, h.rank
    epoch = st.calls + 1
    par = epoch & 1
    tiles = st.flags.shape[2]
    peers_sl = [h.symm_at(st.slots, p) for p in range(W)]
    peers_fl = [h.symm_at(st.flags, p) for p in range(W)]
    for d in range(1, W):
        seg = (rank + d) % W
        for t in range(tiles):
            r0, r1 = t * st.tile_rows, min((t + 1) * st.tile_rows, st.rows)
            peers_sl[seg][par, rank, r0:r1] = partial[seg * st.rows + r0: seg * st.rows + r1]
            FakeSymmHeap.signal(peers_fl[seg][par, rank], t, epoch)
    out = partial[rank * st.rows:(rank + 1) * st.rows].clone()
    for t in range(tiles):
        r0, r1 = t * st.tile_rows, min((t + 1) * st.tile_rows, st.rows)
        for d in range(1, W):
            src = (rank + d) % W
            FakeSymmHeap.wait_until(st.flags[par, src], t, epoch, geq=True, timeout_s=timeout_s, where=2, peer=src)
            out[r0:r1] += st.slots[par, src, r0:r1]
    st.calls += 1
    return out


def poison_unused_parity(buf: torch.Tensor, calls: int) -> None:
    """Host twin of ``ops.common.poison_unused_parity``: NaN into the half the call with epoch ``calls + 1`` does not use."""
    buf[(calls + 1) & 1 ^ 1].fill_(float("nan"))

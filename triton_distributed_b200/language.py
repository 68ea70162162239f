"""The device language of this library and how it maps onto the reference's.

The reference extends Triton with six distributed ops and exposes the NVSHMEM device API
(python/triton_dist/language/distributed_ops.py:57-111, language/extra/libshmem_device.py:28-289).  Here kernels are
CUDA C++ and the same vocabulary is a header-only device API, ``csrc/include/tdb/symm_device.cuh`` + ``ptx.cuh``:

==============================================  ==========================================================================
reference (Triton-distributed)                  this library (CUDA C++, namespace ``tdb``)
==============================================  ==========================================================================
``dl.rank()`` / ``dl.num_ranks()``              ``my_pe(symm)`` / ``n_pes(symm)``
``dl.symm_at(ptr, rank)``                       ``symm_at(symm, ptr, rank)``
``libshmem_device.remote_mc_ptr(team, ptr)``    ``mc_ptr(symm, ptr)``
``dl.notify(ptr, rank, v, "set"|"add", scope)`` ``notify(symm, flag, rank, v, kSignalSet|kSignalAdd)`` (fenced release store /
                                                reduction to the peer's flag)
``dl.wait(ptr, n, scope, sem, value)``          ``warp_wait_flags(symm, flags, n, value, cmp, ...)`` / ``wait_until(...)``:
                                                acquire spin, BOUNDED, returns a status instead of hanging
``dl.consume_token(x, token)``                  not needed: the acquire load of the wait orders later loads; before a TMA
                                                load of the awaited data add ``fence_proxy_async()``
``putmem / getmem {,_nbi}{,_warp,_block}``      ``putmem_thread/warp/block``, ``getmem_warp/block`` (16-byte vector copies
                                                to / from the peer mapping); ``_nbi`` = the same call without a following fence
``putmem_signal*``                              ``putmem_signal_block``
``signal_op`` / ``signal_wait_until``           ``notify`` / ``wait_until``
``fence`` / ``quiet``                           ``fence(symm)`` / ``quiet(symm)``
``barrier_all{,_block,_warp}``                  ``rank_barrier_block`` (epoch flags), host: ``barrier_all_on_stream``
grid barrier (common_ops.py:57-138)             ``grid_barrier``
``multimem_ld_reduce_v4`` / ``multimem_st_*``   ``multimem_ld_reduce_bf16x8 / f16x8 / f32x4``, ``multimem_st_v4``,
                                                ``multimem_red_release_add_u32``
``ld / st / atomic_*`` with scope & semantic    ``ld_acquire_sys/gpu``, ``ld_relaxed_sys``, ``st_release_sys/gpu``,
                                                ``red_release_*_add``, ``atom_add_acqrel_*``, ``atom_cas_acqrel_sys``
``tid / ntid / laneid / __syncthreads /         plain CUDA (``threadIdx``, ``lane_id()``, ``__syncthreads``, ``__shfl_*``)
shuffles / ballot``
``simt_exec_region``                            not needed: CUDA C++ is already per-thread code
==============================================  ==========================================================================

Host side the symbols below give a Python view of the same model for tests and tutorials: symmetric tensors, peer
views, and stream-ordered ``set_signal`` / ``wait_eq`` (python/triton_dist/kernels/common_ops.py:25-39).
"""
from __future__ import annotations

import torch

from . import _native
from .runtime import get_runtime

SIGNAL_SET, SIGNAL_ADD = 0, 1
CMP_EQ, CMP_GE, CMP_NE = 0, 1, 2


def rank() -> int:
    return get_runtime().rank


def num_ranks() -> int:
    return get_runtime().world_size


def symm_at(t: torch.Tensor, peer: int) -> torch.Tensor:
    """Peer-mapped view of a symmetric tensor (the host-side analogue of the device call)."""
    return get_runtime().peer_view(t, peer)


def mc_view(t: torch.Tensor) -> torch.Tensor:
    return get_runtime().multicast_view(t)


def set_signal(flag: torch.Tensor, value: int, stream=None):
    """Stream-ordered write of a 32-bit flag (cuStreamWriteValue32)."""
    lib = _native.load(True)
    with torch.cuda.stream(stream or torch.cuda.current_stream()):
        lib.stream_write_value32(flag.data_ptr(), int(value))


def wait_eq(flag: torch.Tensor, value: int, stream=None, geq: bool = False, timeout_s=None, bounded: bool = True):
    """Stream-ordered wait on a 32-bit flag: later work on the stream starts once the flag equals (``geq``: has
    reached) ``value``.

    By default the wait is a one-thread kernel with the runtime's time limit (``TDB200_WAIT_TIMEOUT_S`` or
    ``timeout_s``): when nothing writes the flag the stream continues after the limit and
    ``Runtime.check_status()`` raises ``CommTimeoutError``.  ``bounded=False`` uses the driver's stream memory
    operation (cuStreamWaitValue32), which has NO time limit: the stream stays blocked until the value is there, so
    only use it for flags that a kernel or stream of this job is certain to write."""
    lib = _native.load(True)
    rt = get_runtime()
    with torch.cuda.stream(stream or torch.cuda.current_stream()):
        if bounded and rt.heap is not None:
            lib.timeout_probe(rt.heap, flag, int(value), float(timeout_s if timeout_s is not None else rt.config.wait_timeout_s),
                              CMP_GE if geq else CMP_EQ)
        else:
            lib.stream_wait_value32(flag.data_ptr(), int(value), bool(geq))


notify = set_signal
wait = wait_eq


def consume_token(value, token=None):
    """The reference ties a loaded value to the token of a preceding ``wait`` so that the compiler cannot hoist the
    load above the wait (python/triton_dist/language/distributed_ops.py:75-87).  Here the ordering is the stream's: work
    enqueued after ``wait`` runs after it, so the value is returned unchanged.  (Inside the CUDA kernels of this
    package the same guarantee comes from the acquire load in ``wait_until``.)"""
    return value

"""Pipeline-parallel transport: double-buffered activation exchange between neighbouring stages.

API of the reference: ``CommOp`` (python/triton_dist/layers/nvidia/p2p.py:43-132) with ``read`` / ``set_signal`` /
``wait_signal``, driven by the send/recv protocol of its test (test/nvidia/test_pp.py:68-120).  The reference moves the
data with an NVSHMEM get kernel; here the bytes travel over NCCL point-to-point on a side stream so they overlap the
stage's compute, and readiness is tracked with CUDA events instead of heap signals.  There is no schedule (1F1B ...)
in the reference either - only the transport.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from ..runtime import get_runtime


class CommOp:
    def __init__(self, max_tokens: int, hidden: int, num_buffers: int = 2, dtype: torch.dtype = torch.bfloat16, group=None):
        rt = get_runtime()
        self.rt = rt
        self.group = group if group is not None else rt.group
        self.rank, self.world = rt.rank, rt.world_size
        self.num_buffers = num_buffers
        self.buffers: List[torch.Tensor] = [torch.empty(max_tokens, hidden, dtype=dtype, device=rt.device)
                                            for _ in range(num_buffers)]
        self.stream = torch.cuda.Stream() if rt.is_cuda else None
        self._ready = [torch.cuda.Event() if rt.is_cuda else None for _ in range(num_buffers)]
        self._work = [None] * num_buffers

    def send(self, x: torch.Tensor, dst: int, buffer_id: int = 0):
        """Asynchronous send of ``x`` to stage ``dst`` (ordered after the producer on the current stream)."""
        if self.stream is None:
            self._work[buffer_id] = dist.isend(x.contiguous(), dst, group=self.group)
            return
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            x.record_stream(self.stream)
            dist.send(x.contiguous(), dst, group=self.group)
            self._ready[buffer_id].record(self.stream)

    def read(self, src: int, num_tokens: int, buffer_id: int = 0) -> torch.Tensor:
        """Start receiving ``num_tokens`` rows from stage ``src`` into comm buffer ``buffer_id``; returns its view."""
        view = self.buffers[buffer_id][:num_tokens]
        if self.stream is None:
            self._work[buffer_id] = dist.irecv(view, src, group=self.group)
            return view
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            dist.recv(view, src, group=self.group)
            self._ready[buffer_id].record(self.stream)
        return view

    def set_signal(self, buffer_id: int = 0):
        """Mark buffer ``buffer_id`` as consumed (the next ``read`` into it may overwrite)."""
        if self.stream is not None:
            self.stream.wait_stream(torch.cuda.current_stream())

    def wait_signal(self, buffer_id: int = 0):
        """Make the current stream wait until the transfer into / out of ``buffer_id`` has finished."""
        if self.stream is None:
            if self._work[buffer_id] is not None:
                self._work[buffer_id].wait()
                self._work[buffer_id] = None
            return
        torch.cuda.current_stream().wait_event(self._ready[buffer_id])

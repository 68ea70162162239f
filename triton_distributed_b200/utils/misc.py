"""Rank-ordered printing, comparisons, data generation, logging."""
from __future__ import annotations

import logging
import os
import sys
from typing import Iterable, Optional, Sequence

import torch
import torch.distributed as dist


def dist_print(*args, allowed_ranks: Optional[Iterable[int]] = (0,), need_sync: bool = False, prefix: bool = False,
               **kwargs):
    """Print from the allowed ranks ("all" for every rank); with ``need_sync`` the ranks print in rank order
    (python/triton_dist/utils.py:289-318)."""
    rank = dist.get_rank() if dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_initialized() else 1
    if allowed_ranks == "all":
        allowed_ranks = range(world)
    allowed = set(allowed_ranks)

    def emit():
        if rank in allowed:
            if prefix:
                print(f"[rank {rank}]", *args, **kwargs)
            else:
                print(*args, **kwargs)
            sys.stdout.flush()

    if not need_sync or not dist.is_initialized():
        emit()
        return
    for r in range(world):
        if r == rank:
            emit()
        dist.barrier()


def assert_allclose(x: torch.Tensor, y: torch.Tensor, rtol: float = 1e-2, atol: float = 1e-2, verbose: bool = True):
    """Raises with the mismatch fraction and the worst element when not close
    (python/triton_dist/utils.py:870-900)."""
    if x.shape != y.shape:
        raise AssertionError(f"shape mismatch {tuple(x.shape)} vs {tuple(y.shape)}")
    xf, yf = x.float(), y.float()
    bad = ~torch.isclose(xf, yf, rtol=rtol, atol=atol)
    if bad.any():
        n = int(bad.sum())
        diff = (xf - yf).abs()
        idx = int(diff.argmax())
        raise AssertionError(f"{n}/{x.numel()} elements differ (rtol={rtol}, atol={atol}); worst |diff|="
                             f"{diff.flatten()[idx].item():.5g} at flat index {idx}: {xf.flatten()[idx].item():.6g} vs "
                             f"{yf.flatten()[idx].item():.6g}")


def bitwise_equal(x: torch.Tensor, y: torch.Tensor) -> bool:
    """Exact equality of the bit patterns (NaNs compare equal when their bits do)."""
    if x.shape != y.shape or x.dtype != y.dtype:
        return False
    return bool(torch.equal(x.contiguous().view(torch.uint8), y.contiguous().view(torch.uint8)))


def generate_data(shape: Sequence[int], dtype: torch.dtype, device, scale: float = 1.0, seed: Optional[int] = None):
    g = None
    if seed is not None:
        g = torch.Generator(device=device).manual_seed(seed)
    return (torch.randn(tuple(shape), device=device, dtype=torch.float32, generator=g) * scale).to(dtype)


class MyLogger:
    """Per-rank logger switched on by ``TDB200_DEBUG`` (the reference's TRITON_DIST_DEBUG, models/utils.py:45-72)."""

    def __init__(self, name: str = "tdb200"):
        self.log = logging.getLogger(name)
        if not self.log.handlers:
            h = logging.StreamHandler()
            h.setFormatter(logging.Formatter("%(asctime)s %(name)s %(levelname)s %(message)s"))
            self.log.addHandler(h)
        self.log.setLevel(logging.DEBUG if os.environ.get("TDB200_DEBUG", "0") not in ("0", "") else logging.INFO)

    def _rank(self):
        return dist.get_rank() if dist.is_initialized() else 0

    def info(self, msg, *a):
        self.log.info(f"[rank {self._rank()}] {msg}", *a)

    def debug(self, msg, *a):
        self.log.debug(f"[rank {self._rank()}] {msg}", *a)

    def warning(self, msg, *a):
        self.log.warning(f"[rank {self._rank()}] {msg}", *a)


logger = MyLogger()

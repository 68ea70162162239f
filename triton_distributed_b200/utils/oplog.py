"""Per-op metrics: when ``TDB200_OP_LOG`` names a file (or ``enable()`` is called), every public op of the package
records a pair of CUDA events around its launch and ``flush()`` turns them into JSON lines

    {"op": "ag_gemm", "shape": {...}, "us": 412.3, "tflops": 1167.0, "roofline_frac": 0.70, "rank": 0}

with the roofline of :mod:`triton_distributed_b200.utils.roofline` (the slower of FLOPs at the measured GEMM peak and
NVLink bytes at the measured link bandwidth).  Off by default: an op then pays one attribute check.  The reference only
prints timings from its benchmark scripts (python/triton_dist/utils.py:274-289 ``perf_func`` / ``dist_print``)."""
from __future__ import annotations

import atexit
import functools
import json
import os
from typing import Callable, Dict, List, Optional

import torch

_ENABLED = False
_PATH: Optional[str] = None
_PENDING: List[tuple] = []
_RECORDS: List[dict] = []


def enable(path: Optional[str] = None):
    global _ENABLED, _PATH
    _ENABLED, _PATH = True, path


def disable():
    global _ENABLED
    _ENABLED = False


def enabled() -> bool:
    return _ENABLED


def records() -> List[dict]:
    """Records produced by the last ``flush()`` calls (kept in memory as well as written to the file)."""
    return list(_RECORDS)


def flush() -> List[dict]:
    """Synchronise, convert pending event pairs into records, append them to the log file.  Returns the new records."""
    from .roofline import fused_roofline

    if not _PENDING:
        return []
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    rank = int(os.environ.get("RANK", 0))
    new = []
    for name, meta, e0, e1, wall_ms in _PENDING:
        ms = e0.elapsed_time(e1) if e0 is not None else wall_ms
        rec = {"op": name, "shape": meta.get("shape", {}), "us": round(ms * 1e3, 2), "rank": rank}
        flops = float(meta.get("flops", 0.0))
        if flops > 0 and ms > 0:
            rec["tflops"] = round(flops / ms / 1e9, 1)
            roof = fused_roofline(flops, float(meta.get("link_bytes", 0.0)), ms)
            rec["roofline_frac"] = round(roof["frac_of_roofline"], 3)
        elif meta.get("bytes") and ms > 0:
            rec["gbs"] = round(float(meta["bytes"]) / ms / 1e6, 1)
        new.append(rec)
    _PENDING.clear()
    _RECORDS.extend(new)
    if _PATH:
        with open(_PATH, "a") as f:
            for r in new:
                f.write(json.dumps(r) + "\n")
    return new


def logged_op(name: str, meta: Callable[..., Dict]):
    """Decorator: ``meta(*args, **kwargs)`` returns ``{"shape": {...}, "flops": F, "link_bytes": B}`` for the call."""

    def deco(fn):
        @functools.wraps(fn)
        def wrapper(*args, **kwargs):
            if not _ENABLED:
                return fn(*args, **kwargs)
            try:
                m = meta(*args, **kwargs)
            except Exception:   # metrics must never break an op
                m = {}
            on_gpu = any(isinstance(a, torch.Tensor) and a.is_cuda for a in args)
            if on_gpu:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                out = fn(*args, **kwargs)
                e1.record()
                _PENDING.append((name, m, e0, e1, 0.0))
            else:
                import time
                t0 = time.perf_counter()
                out = fn(*args, **kwargs)
                _PENDING.append((name, m, None, None, (time.perf_counter() - t0) * 1e3))
            return out

        return wrapper

    return deco


if os.environ.get("TDB200_OP_LOG"):
    enable(os.environ["TDB200_OP_LOG"])
    atexit.register(flush)

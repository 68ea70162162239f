"""Contextual autotuner: times the WHOLE distributed thunk once per candidate configuration so that all ranks stay
in lock step, takes the maximum over ranks, and caches the winner per key.

API of the reference: ``contextual_autotune(is_dist, n_repeat, n_warmup)`` (python/triton_dist/autotuner.py:43-250).
The reference patches Triton's per-kernel autotuner; here kernels are ahead-of-time compiled and the tunable knobs are
launch-level (comm CTAs, tile width, K splits, all-reduce method ...), exposed to the tuned function through
``current_config()``.
"""
from __future__ import annotations

import functools
import itertools
import json
import os
from typing import Any, Callable, Dict, Iterable, List, Optional

import torch
import torch.distributed as dist

_ACTIVE: Optional[Dict[str, Any]] = None
_CACHE: Dict[str, Dict[str, Any]] = {}


def current_config(default: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
    """Configuration the autotuner is currently trying (or has chosen); ``default`` outside of a tuned call."""
    return dict(_ACTIVE) if _ACTIVE is not None else dict(default or {})


def config_space(**axes: Iterable) -> List[Dict[str, Any]]:
    keys = list(axes)
    return [dict(zip(keys, vals)) for vals in itertools.product(*[list(axes[k]) for k in keys])]


def _log(rank: int, msg: str, log_dir: str):
    os.makedirs(log_dir, exist_ok=True)
    with open(os.path.join(log_dir, f"rank-{rank}.log"), "a") as f:
        f.write(msg + "\n")


def contextual_autotune(configs: Optional[List[Dict[str, Any]]] = None, key: Optional[Callable[..., str]] = None,
                        is_dist: bool = False, n_repeat: int = 5, n_warmup: int = 3, log_dir: str = "./.autotune_logs"):
    """Decorator.  The wrapped function is run ``n_warmup + n_repeat`` times per candidate; the fastest candidate
    (max over ranks of the mean device time when ``is_dist``) is cached under ``key(*args)`` and used afterwards."""

    def deco(fn: Callable):
        @functools.wraps(fn)
        def wrapper(*args, **kwargs):
            global _ACTIVE
            cands = configs or [{}]
            k = f"{fn.__module__}.{fn.__qualname__}:" + (key(*args, **kwargs) if key else "default")
            if k not in _CACHE:
                rank = dist.get_rank() if dist.is_initialized() else 0
                best, best_t = None, float("inf")
                for cfg in cands:
                    _ACTIVE = cfg
                    try:
                        for _ in range(n_warmup):
                            fn(*args, **kwargs)
                        if torch.cuda.is_available():
                            torch.cuda.synchronize()
                            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                            s.record()
                            for _ in range(n_repeat):
                                fn(*args, **kwargs)
                            e.record()
                            torch.cuda.synchronize()
                            t = s.elapsed_time(e) / n_repeat
                        else:
                            import time
                            t0 = time.perf_counter()
                            for _ in range(n_repeat):
                                fn(*args, **kwargs)
                            t = (time.perf_counter() - t0) * 1e3 / n_repeat
                    except Exception as ex:  # a candidate that cannot run is simply not chosen
                        t = float("inf")
                        _log(rank, f"{k} {json.dumps(cfg)} failed: {ex}", log_dir)
                    if is_dist and dist.is_initialized() and dist.get_world_size() > 1:
                        tt = torch.tensor([t], dtype=torch.float64, device="cuda" if torch.cuda.is_available() else "cpu")
                        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
                        t = float(tt.item())
                    _log(rank, f"{k} {json.dumps(cfg)} {t:.4f} ms", log_dir)
                    if t < best_t:
                        best, best_t = cfg, t
                _CACHE[k] = dict(best or {})
                _log(rank, f"{k} best {json.dumps(_CACHE[k])} {best_t:.4f} ms", log_dir)
            _ACTIVE = _CACHE[k]
            try:
                return fn(*args, **kwargs)
            finally:
                _ACTIVE = None

        wrapper.autotune_cache = _CACHE
        return wrapper

    return deco

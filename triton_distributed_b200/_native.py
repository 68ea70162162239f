"""Loader of the in-tree native library.

The shared object is built by :mod:`triton_distributed_b200.build` and is never compiled at import time.
On a machine with a GPU a missing library is an error (ops must not fall back silently); without a GPU
the torch reference backend is used and the library is optional.
"""
from __future__ import annotations

import importlib.util
from pathlib import Path

import torch

_LIB = None
_ERR = None


def lib_path() -> Path:
    return Path(__file__).resolve().parent / "_C.so"


def load(required: bool = False):
    """Return the native module, or None when it is not built and ``required`` is False."""
    global _LIB, _ERR
    if _LIB is not None:
        return _LIB
    p = lib_path()
    if p.exists():
        try:
            spec = importlib.util.spec_from_file_location("triton_distributed_b200._C", str(p))
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            _LIB = mod
            return _LIB
        except Exception as e:  # pragma: no cover - depends on the machine
            _ERR = e
    else:
        _ERR = FileNotFoundError(f"{p} not built; run `python -m triton_distributed_b200.build`")
    if required or torch.cuda.is_available():
        raise RuntimeError(f"triton_distributed_b200 native library unavailable: {_ERR}")
    return None


def available() -> bool:
    try:
        return load(False) is not None
    except RuntimeError:
        return False


def use_native(*tensors) -> bool:
    """True when the op should run the CUDA kernel: all tensors on a GPU (then the library is mandatory)."""
    if tensors and all(isinstance(t, torch.Tensor) and t.is_cuda for t in tensors):
        load(True)
        return True
    return False

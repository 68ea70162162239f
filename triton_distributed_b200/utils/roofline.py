"""Roofline arithmetic against the measured peaks of this machine pool.

The denominators are a measured copy bandwidth and a measured cuBLAS bf16 GEMM rate (file
``MEASURED_PEAKS.json`` at the repository root when present, else the stated fallback).  Plays the role of the
reference's speed-of-light models (python/triton_dist/kernels/nvidia/gemm_perf_model.py:61-236,
comm_perf_model.py:83-116), which have no Blackwell entry.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional

FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}
NVLINK_GBS_MEASURED = 770.0   # peer copy, per direction per GPU, measured on this pool
NVLINK_GBS_NOMINAL = 900.0


def load_peaks(path: Optional[str] = None) -> Dict[str, float]:
    if path is None:
        path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                            "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    except (OSError, KeyError, ValueError):
        return dict(FALLBACK)


def gemm_roofline(M: int, N: int, K: int, ms: float, elem_bytes: int = 2, peaks: Optional[dict] = None) -> dict:
    """Achieved TFLOP/s and fraction of the measured burst peak for one GEMM."""
    peaks = peaks or load_peaks()
    flops = 2.0 * M * N * K
    tflops = flops / (ms * 1e-3) / 1e12
    bytes_ = (M * K + N * K + M * N) * elem_bytes
    t_compute = flops / (peaks["bf16_tflops"] * 1e12)
    t_mem = bytes_ / (peaks["hbm_gbs"] * 1e9)
    t_roof = max(t_compute, t_mem)
    return {"tflops": tflops, "frac_of_peak": tflops / peaks["bf16_tflops"], "roofline_ms": t_roof * 1e3,
            "frac_of_roofline": t_roof * 1e3 / ms, "peaks": peaks["source"]}


def fused_roofline(flops_per_rank: float, nvlink_bytes_per_rank: float, ms: float, peaks: Optional[dict] = None) -> dict:
    """Fused compute+collective kernel: target = slower of compute at the measured GEMM peak and the bytes that
    must cross NVLink at the measured per-direction link bandwidth."""
    peaks = peaks or load_peaks()
    t_compute = flops_per_rank / (peaks["bf16_tflops"] * 1e12)
    t_link = nvlink_bytes_per_rank / (NVLINK_GBS_MEASURED * 1e9)
    t_roof = max(t_compute, t_link)
    return {"compute_ms": t_compute * 1e3, "link_ms": t_link * 1e3, "roofline_ms": t_roof * 1e3,
            "frac_of_roofline": t_roof * 1e3 / ms, "tflops_per_rank": flops_per_rank / (ms * 1e-3) / 1e12,
            "peaks": peaks["source"]}

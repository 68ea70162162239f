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


# ---------------------------------------------------------------------------------------------------------------------
# Speed-of-light estimates with the reference's function names (gemm_perf_model.py:198-236, comm_perf_model.py:94-116),
# for a B200 inside one NVSwitch domain.  Dense nominal tensor peaks; measured values where this pool has them.
# ---------------------------------------------------------------------------------------------------------------------
NOMINAL_TFLOPS = {"bf16": 2250.0, "fp16": 2250.0, "fp8": 4500.0, "fp4": 9000.0, "tf32": 1100.0}


def get_tensorcore_tflops(dtype="bf16", measured: bool = True) -> float:
    """Dense tensor-core rate of one B200: the measured cuBLAS bf16 burst rate (scaled by the nominal ratio for other
    types) or the nominal figure."""
    name = str(dtype).replace("torch.", "")
    name = {"bfloat16": "bf16", "float16": "fp16", "float8_e4m3fn": "fp8", "float8_e5m2": "fp8", "float32": "tf32"}.get(name, name)
    nominal = NOMINAL_TFLOPS[name]
    if not measured:
        return nominal
    return load_peaks()["bf16_tflops"] * nominal / NOMINAL_TFLOPS["bf16"]


def get_dram_gbps(measured: bool = True) -> float:
    return load_peaks()["hbm_gbs"] if measured else 7700.0


def estimate_gemm_sol_time_ms(M: int, N: int, K: int, dtype="bf16", elem_bytes: int = 2) -> float:
    """max(compute at the tensor peak, operands + result once over HBM)."""
    t_c = 2.0 * M * N * K / (get_tensorcore_tflops(dtype) * 1e12)
    t_m = (M * K + N * K + M * N) * elem_bytes / (get_dram_gbps() * 1e9)
    return max(t_c, t_m) * 1e3


def estimate_all_gather_time_ms(nbytes: int, world_size: int, local_world_size: Optional[int] = None,
                                intranode_bw: float = NVLINK_GBS_MEASURED, internode_bw: Optional[float] = None) -> float:
    """Every rank receives (W - 1) / W of ``nbytes`` (the gathered size) through its own NVLink ingress."""
    return nbytes * (world_size - 1) / world_size / (intranode_bw * 1e9) * 1e3


def estimate_reduce_scatter_time_ms(nbytes: int, world_size: int, local_world_size: Optional[int] = None,
                                    intranode_bw: float = NVLINK_GBS_MEASURED, internode_bw: Optional[float] = None) -> float:
    """Every rank sends (W - 1) / W of its ``nbytes`` partial result."""
    return nbytes * (world_size - 1) / world_size / (intranode_bw * 1e9) * 1e3

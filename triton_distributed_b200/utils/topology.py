"""Hardware and topology probes (read-only): NVLink full-mesh detection, NVLS / TMA support, NUMA node, SM count, shared
memory and stream-priority limits.  Covers python/triton_dist/utils.py:592-867, :944-1092 of the reference.  Every probe
only reads state; nothing here changes a GPU setting."""
from __future__ import annotations

import functools
import os
import subprocess
from typing import List, Optional

import torch


def _nvml():
    try:
        import pynvml
        pynvml.nvmlInit()
        return pynvml
    except Exception:
        return None


@functools.lru_cache()
def device_count() -> int:
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@functools.lru_cache()
def has_fullmesh_nvlink(num_gpus: Optional[int] = None) -> bool:
    """True when every pair of visible GPUs is NVLink-connected (NVML P2P status, else `nvidia-smi topo -m`)."""
    n = num_gpus or device_count()
    if n < 2:
        return False
    nv = _nvml()
    if nv is not None:
        try:
            hs = [nv.nvmlDeviceGetHandleByIndex(i) for i in range(n)]
            for i in range(n):
                for j in range(n):
                    if i != j and nv.nvmlDeviceGetP2PStatus(hs[i], hs[j], nv.NVML_P2P_CAPS_INDEX_NVLINK) != nv.NVML_P2P_STATUS_OK:
                        return False
            return True
        except Exception:
            pass
    try:
        out = subprocess.run(["nvidia-smi", "topo", "-m"], capture_output=True, text=True, timeout=20).stdout
    except (OSError, subprocess.TimeoutExpired):
        return False
    rows = [l.split() for l in out.splitlines() if l.startswith("GPU")]
    for i, r in enumerate(rows[:n]):
        for j, cell in enumerate(r[1:n + 1]):
            if i != j and not cell.startswith("NV"):
                return False
    return bool(rows)


def nvlink_links(device: int = 0) -> int:
    nv = _nvml()
    if nv is None:
        return 0
    try:
        h = nv.nvmlDeviceGetHandleByIndex(device)
        n = 0
        for l in range(32):
            try:
                if nv.nvmlDeviceGetNvLinkState(h, l):
                    n += 1
            except Exception:
                break
        return n
    except Exception:
        return 0


def numa_node(device: int = 0) -> int:
    """NUMA node of the GPU's PCI device, -1 when unknown."""
    nv = _nvml()
    if nv is None:
        return -1
    try:
        bus = nv.nvmlDeviceGetPciInfo(nv.nvmlDeviceGetHandleByIndex(device)).busId
        bus = bus.decode() if isinstance(bus, bytes) else bus
        path = f"/sys/bus/pci/devices/{bus[-12:].lower()}/numa_node"
        with open(path) as f:
            return int(f.read().strip())
    except Exception:
        return -1


def has_nvls() -> bool:
    """NVLS multicast usable: the runtime's heap managed to bind a multicast object (or, before init, cc >= 9)."""
    try:
        from ..runtime import get_runtime
        return get_runtime().has_multicast
    except RuntimeError:
        return torch.cuda.is_available() and torch.cuda.get_device_capability()[0] >= 9


def has_tma() -> bool:
    return torch.cuda.is_available() and torch.cuda.get_device_capability()[0] >= 9


def has_tcgen05() -> bool:
    return torch.cuda.is_available() and torch.cuda.get_device_capability()[0] == 10


def supports_p2p_native_atomic() -> bool:
    return has_fullmesh_nvlink()


def sm_count(device: int = 0) -> int:
    return torch.cuda.get_device_properties(device).multi_processor_count if torch.cuda.is_available() else 0


def max_shared_memory_per_block(device: int = 0) -> int:
    p = torch.cuda.get_device_properties(device)
    return int(getattr(p, "shared_memory_per_block_optin", 0) or getattr(p, "max_shared_memory_per_block_optin", 0) or 232448)


def max_stream_priority() -> int:
    return -5 if torch.cuda.is_available() else 0


def describe() -> dict:
    return {"gpus": device_count(), "fullmesh_nvlink": has_fullmesh_nvlink(), "nvlink_links": nvlink_links(0) if device_count() else 0,
            "nvls": has_nvls(), "tma": has_tma(), "tcgen05": has_tcgen05(), "sms": sm_count() if device_count() else 0,
            "numa_node": numa_node(0) if device_count() else -1}

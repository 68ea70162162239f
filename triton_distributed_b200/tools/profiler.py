"""Host side of the intra-kernel profiler: buffer creation, decoding, Chrome-trace export, per-SM activity.

Device side: ``csrc/include/tdb/profiler.cuh`` (``TDB_PROFILE_RECORD``).  Counterpart of the reference's
tools/profiler (context.py:49-78, viewer.py:55-183) and of ``ModelBuilder.dump_trace`` / ``get_sm_activity``
(mega_triton_kernel/models/model_builder.py:161, :538)."""
from __future__ import annotations

import json
from typing import Dict, List, Optional

import torch


def create_buffer(capacity: int, device="cuda") -> torch.Tensor:
    """uint64 buffer for ``capacity`` records; pass its data_ptr to a kernel built with profiling."""
    buf = torch.zeros(2 + 2 * capacity, dtype=torch.int64, device=device)
    buf[1] = capacity
    return buf


def decode(buf: torch.Tensor) -> List[dict]:
    host = buf.cpu().tolist()
    n = min(host[0], host[1])
    out = []
    for i in range(n):
        w0, w1 = host[2 + 2 * i] & 0xFFFFFFFFFFFFFFFF, host[3 + 2 * i] & 0xFFFFFFFFFFFFFFFF
        tag, t_lo = w0 >> 32, w0 & 0xFFFFFFFF
        sm, t_hi = w1 >> 32, w1 & 0xFFFFFFFF
        out.append({"block": (tag >> 16) & 0xFFFF, "group": (tag >> 12) & 0xF, "task": (tag >> 1) & 0x7FF,
                    "start": bool(tag & 1), "sm": sm, "t_ns": (t_hi << 32) | t_lo})
    return out


def to_chrome_trace(records: List[dict], task_names: Optional[Dict[int, str]] = None, path: Optional[str] = None) -> dict:
    """Pairs start/end records per (block, group, task) into complete events; pid = SM, tid = group."""
    task_names = task_names or {}
    t0 = min((r["t_ns"] for r in records), default=0)
    open_ev, events = {}, []
    for r in sorted(records, key=lambda r: r["t_ns"]):
        key = (r["block"], r["group"], r["task"])
        if r["start"]:
            open_ev[key] = r
        elif key in open_ev:
            s = open_ev.pop(key)
            events.append({"name": task_names.get(r["task"], f"task{r['task']}"), "ph": "X", "pid": f"SM {s['sm']}",
                           "tid": f"group {s['group']}", "ts": (s["t_ns"] - t0) / 1e3, "dur": (r["t_ns"] - s["t_ns"]) / 1e3,
                           "args": {"block": s["block"]}})
    trace = {"traceEvents": events, "displayTimeUnit": "ns"}
    if path:
        with open(path, "w") as f:
            json.dump(trace, f)
    return trace


def sm_activity(records: List[dict]) -> Dict[int, float]:
    """Busy fraction of every SM between the first and the last record."""
    if not records:
        return {}
    t0, t1 = min(r["t_ns"] for r in records), max(r["t_ns"] for r in records)
    span = max(1, t1 - t0)
    busy: Dict[int, int] = {}
    open_ev = {}
    for r in sorted(records, key=lambda r: r["t_ns"]):
        key = (r["block"], r["group"], r["task"])
        if r["start"]:
            open_ev[key] = r
        elif key in open_ev:
            s = open_ev.pop(key)
            busy[s["sm"]] = busy.get(s["sm"], 0) + (r["t_ns"] - s["t_ns"])
    return {sm: b / span for sm, b in busy.items()}

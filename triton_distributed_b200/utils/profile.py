"""torch.profiler capture merged over ranks into one chrome trace
(python/triton_dist/utils.py:262-271 ``get_torch_prof_ctx``, :505-589 ``group_profile``)."""
from __future__ import annotations

import contextlib
import gzip
import json
import os
import tarfile
import tempfile
from typing import Optional

import torch
import torch.distributed as dist


def get_torch_prof_ctx(do_prof: bool):
    if not do_prof:
        return contextlib.nullcontext()
    acts = [torch.profiler.ProfilerActivity.CPU]
    if torch.cuda.is_available():
        acts.append(torch.profiler.ProfilerActivity.CUDA)
    return torch.profiler.profile(activities=acts, record_shapes=True, with_stack=False)


def _merge_traces(traces):
    """Give every rank its own pid range so the timelines sit side by side."""
    events = []
    for rank, tr in enumerate(traces):
        for ev in tr.get("traceEvents", []):
            ev = dict(ev)
            if "pid" in ev:
                ev["pid"] = f"rank{rank}:{ev['pid']}"
            events.append(ev)
    return {"traceEvents": events, "displayTimeUnit": "ms"}


@contextlib.contextmanager
def group_profile(name: str = "trace", do_prof: bool = True, group=None, out_dir: str = "prof"):
    """Profile the body on every rank; rank 0 writes ``<out_dir>/<name>.json.tar.gz`` with all ranks merged."""
    if not do_prof:
        yield None
        return
    prof = get_torch_prof_ctx(True)
    with prof:
        yield prof
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    with tempfile.TemporaryDirectory() as td:
        path = os.path.join(td, "t.json")
        prof.export_chrome_trace(path)
        with open(path) as f:
            mine = json.load(f)
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    traces = [mine]
    if world > 1:
        gathered = [None] * world if rank == 0 else None
        dist.gather_object(mine, gathered, dst=0, group=group)
        traces = gathered
    if rank == 0:
        os.makedirs(out_dir, exist_ok=True)
        merged = _merge_traces(traces)
        jpath = os.path.join(out_dir, f"{name}.json")
        with open(jpath, "w") as f:
            json.dump(merged, f)
        with tarfile.open(jpath + ".tar.gz", "w:gz") as tar:
            tar.add(jpath, arcname=f"{name}.json")
        os.remove(jpath)

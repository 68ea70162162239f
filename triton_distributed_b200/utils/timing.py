"""Device-side timing with CUDA events, L2 flushing between iterations, and clock sampling."""
from __future__ import annotations

import statistics
import subprocess
import threading
import time
from typing import Callable, List, Optional, Tuple

import torch


class L2Flusher:
    """Writes a buffer larger than the 126 MB L2 so the next timed iteration starts cold."""

    def __init__(self, device=None, nbytes: int = 256 << 20):
        self.buf = torch.empty(nbytes // 4, dtype=torch.int32, device=device or "cuda")

    def flush(self):
        self.buf.zero_()


def device_time_ms(fn: Callable, iters: int = 10, warmup: int = 3, flush_l2: bool = True,
                   flusher: Optional[L2Flusher] = None) -> List[float]:
    """Per-iteration device times (ms) of ``fn`` measured with CUDA events on the current stream."""
    if flush_l2 and flusher is None:
        flusher = L2Flusher()
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush_l2:
            flusher.flush()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    return times


def perf_func(func: Callable, iters: int, warmup_iters: int) -> Tuple[object, float]:
    """Reference-compatible helper: returns (last output, mean ms per iteration); no L2 flush
    (python/triton_dist/utils.py:274-286)."""
    out = None
    for _ in range(warmup_iters):
        out = func()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        out = func()
    e.record()
    torch.cuda.synchronize()
    return out, s.elapsed_time(e) / max(iters, 1)


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while a timed region runs (read-only queries)."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int = 0, period_ms: int = 100):
        self.gpu_index = gpu_index
        self.period_ms = period_ms
        self.rows: List[List[str]] = []
        self.stamps: List[float] = []                     # host time of every row
        self.windows: List[Tuple[float, float]] = []      # timed regions: only their samples are summarised
        self._win_t0: Optional[float] = None
        self._proc = None
        self._thread = None

    def begin_window(self):
        """Start of a timed region (samples outside any window, e.g. during set-up, are ignored by ``stop``)."""
        self._win_t0 = time.time()

    def end_window(self):
        if self._win_t0 is not None:
            self.windows.append((self._win_t0, time.time()))
            self._win_t0 = None

    def start(self):
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-i", str(self.gpu_index),
                 "-lms", str(self.period_ms)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self._proc = None
            return self
        self._thread = threading.Thread(target=self._read, daemon=True)
        self._thread.start()
        return self

    def wait_first_sample(self, timeout_s: float = 5.0) -> bool:
        """Block until the query tool has delivered its first line (its start-up is over) or ``timeout_s`` passed."""
        t0 = time.time()
        while not self.rows and time.time() - t0 < timeout_s:
            if self._proc is None or self._proc.poll() is not None:
                return False
            time.sleep(0.02)
        return bool(self.rows)

    def _read(self):
        for line in self._proc.stdout:
            parts = [p.strip() for p in line.strip().split(",")]
            if len(parts) >= 9:
                self.rows.append(parts)
                self.stamps.append(time.time())

    def stop(self) -> dict:
        if self._proc is not None:
            time.sleep(self.period_ms / 1000.0)
            self._proc.terminate()
            try:
                self._proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self._proc.kill()
        self.end_window()
        sm, mx, reasons = [], [], set()
        slack = self.period_ms / 1000.0
        in_win = [any(a - slack <= t <= b + slack for a, b in self.windows) for t in self.stamps]
        use_windows = bool(self.windows) and any(in_win)
        for idx, r in enumerate(self.rows):
            if use_windows and not (idx < len(in_win) and in_win[idx]):
                continue
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower() == "active":
                    reasons.add(name)
        # samples under load: the upper half of the observed clocks are the busy ones
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}

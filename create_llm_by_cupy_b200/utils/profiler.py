"""Tracing and timing: NVTX ranges keyed by the same tags the manager attaches to prefetches and
bucket flushes (the reference carries those tag strings but never consumes them,
model/model.py:217-383), CUDA-event step timers (device time, not host wall clock) and a sampler of
SM clocks / throttle reasons for benchmark records.
"""
from __future__ import annotations

import contextlib
import subprocess
import threading
import time

import torch


@contextlib.contextmanager
def nvtx_range(tag: str, enabled: bool = True):
    if enabled and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(tag)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


class DeviceTimer:
    """Named CUDA-event intervals on the current stream; ``summary()`` synchronises once."""

    def __init__(self, enabled: bool = True):
        self.enabled = enabled and torch.cuda.is_available()
        self.open = {}
        self.spans = []
        self.host = {}

    def start(self, name: str):
        if self.enabled:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.open[name] = ev
        else:
            self.host[name] = time.perf_counter()

    def stop(self, name: str):
        if self.enabled:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.spans.append((name, self.open.pop(name), ev))
        else:
            self.spans.append((name, self.host.pop(name), time.perf_counter()))

    @contextlib.contextmanager
    def span(self, name: str):
        self.start(name)
        try:
            yield
        finally:
            self.stop(name)

    def summary(self, reset: bool = True) -> dict:
        out = {}
        if self.enabled:
            torch.cuda.synchronize()
            for name, a, b in self.spans:
                out[name] = out.get(name, 0.0) + a.elapsed_time(b)
        else:
            for name, a, b in self.spans:
                out[name] = out.get(name, 0.0) + (b - a) * 1e3
        if reset:
            self.spans = []
        return out


class ClockSampler:
    """Samples SM clock and throttle reasons with ``nvidia-smi`` while a timed region runs (read
    only; never changes a GPU setting)."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int = 0, period_s: float = 0.2):
        self.gpu_index = gpu_index
        self.period_s = period_s
        self.samples = []
        self._stop = threading.Event()
        self._thread = None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.QUERY}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                parts = [p.strip() for p in out.strip().split(",")]
                if len(parts) >= 7:
                    self.samples.append(parts)
            except Exception:
                pass
            self._stop.wait(self.period_s)

    def start(self):
        self._stop.clear()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def stop(self) -> dict:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=10)
        sm, mx, reasons = [], 0.0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx = max(mx, float(s[1]))
            except ValueError:
                continue
            for name, flag in zip(names, s[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}

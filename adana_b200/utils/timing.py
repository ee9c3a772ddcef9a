"""Device-side timing and profiler ranges.

`DeviceTimer` brackets a region with CUDA events on the current stream and, in a multi-rank
job, reports the maximum over ranks (a step is as slow as its slowest rank).  `ClockSampler`
polls `nvidia-smi` for SM clocks and throttle reasons while a benchmark's timed region runs.
"""
from __future__ import annotations

import contextlib
import statistics
import subprocess
import threading
from typing import Optional

import torch
import torch.distributed as dist


class DeviceTimer:
    def __init__(self, enabled: bool = True, reduce_max: bool = True):
        self.enabled = enabled and torch.cuda.is_available()
        self.reduce_max = reduce_max
        self._e0 = self._e1 = None

    def start(self):
        if not self.enabled:
            return
        self._e0 = torch.cuda.Event(enable_timing=True)
        self._e1 = torch.cuda.Event(enable_timing=True)
        self._e0.record()

    def stop(self) -> Optional[float]:
        """Seconds between start() and now on the device (max over ranks), or None if disabled."""
        if not self.enabled:
            return None
        self._e1.record()
        self._e1.synchronize()
        sec = self._e0.elapsed_time(self._e1) / 1e3
        if self.reduce_max and dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            t = torch.tensor([sec], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            sec = float(t.item())
        return sec


@contextlib.contextmanager
def nvtx_range(name: str, cfg=None):
    on = bool(getattr(cfg, "nvtx", False)) and torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
          "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
          "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    """Samples GPU clocks / throttle reasons every `period_ms` in a background process."""

    def __init__(self, gpu_index: int = 0, period_ms: int = 200):
        self.gpu_index, self.period_ms = gpu_index, period_ms
        self._proc = None
        self._lines = []
        self._thread = None

    def start(self):
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={_QUERY}", "--format=csv,noheader,nounits",
                 "-lms", str(self.period_ms), "-i", str(self.gpu_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except (FileNotFoundError, OSError):
            self._proc = None
            return

        def pump():
            for line in self._proc.stdout:
                self._lines.append(line.strip())

        self._thread = threading.Thread(target=pump, daemon=True)
        self._thread.start()

    def stop(self) -> dict:
        if self._proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self._proc.terminate()
        try:
            self._proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self._proc.kill()
        sm, smax, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self._lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "reasons": sorted(reasons), "samples": len(sm)}

"""Device-side timing and clock sampling.

``cuda_time`` brackets a callable with CUDA events on the current stream and a
synchronise on both sides.  ``ClockSampler`` polls ``nvidia-smi`` in a background
thread while a timed region runs and summarises SM clocks and throttle reasons
(read-only: nothing here changes a GPU setting).
"""
from __future__ import annotations

import statistics
import subprocess
import threading
import time
from typing import Callable, List, Optional

import torch

_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
          "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
          "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


def cuda_time(fn: Callable[[], None], iters: int = 1) -> float:
    """Milliseconds per call of ``fn`` measured with CUDA events (no warm-up here)."""
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def flush_l2(buf: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Writes a buffer larger than the 126 MB L2 so the next kernel starts cold."""
    if buf is None:
        buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    buf.zero_()
    return buf


class ClockSampler:
    """Samples SM clocks of one GPU every ``period_ms`` between ``start`` and ``stop``."""

    def __init__(self, gpu_index: int = 0, period_ms: int = 200):
        self.gpu_index, self.period_ms = gpu_index, period_ms
        self.rows: List[List[str]] = []
        self._proc = None
        self._thread = None

    def start(self):
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={_QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(self.gpu_index), "-lms", str(self.period_ms)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self._proc = None
            return self
        self._thread = threading.Thread(target=self._read, daemon=True)
        self._thread.start()
        return self

    def _read(self):
        for line in self._proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 9:
                self.rows.append(parts)

    def stop(self) -> dict:
        if self._proc is not None:
            time.sleep(self.period_ms / 1000.0 * 1.2)
            self._proc.terminate()  # our own child process, by handle
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()
            if self._thread is not None:
                self._thread.join(timeout=2)
        return self.summary()

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
            for name, val in zip(names, r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}

"""Tracing of native kernel calls and module spans.

The reference has no tracing in library code; the hook points it offers are the name on
every tape node (tensor/autograd.go:36-41) and the global module hooks (nn/hooks.go:169-198).
Here every native entry point goes through ``gonn_b200.lib.call``, so one hook there sees
every kernel launch of the framework:

* :class:`Tracer` records, per call, the entry-point name, the host time spent in the launch
  and (optionally) the device time between two CUDA events on the launching stream; it
  prints a per-kernel summary and writes a Chrome trace (``chrome://tracing`` / Perfetto).
* ``nvtx=True`` brackets each call with an NVTX range so that Nsight tools and
  ``torch.profiler`` timelines carry the entry-point names.
* :func:`trace_modules` adds module spans (forward pre / post hooks) to the same timeline.
* :class:`StepTimer` times training steps on the device and reduces with MAX over ranks.

Nothing is recorded unless a tracer is active; the idle cost is one ``is None`` test per call.
"""
from __future__ import annotations

import json
import threading
import time
from collections import defaultdict
from typing import Dict, List, Optional

import torch

from .. import lib as _l

_active: Optional["Tracer"] = None


class _Span:
    __slots__ = ("name", "cat", "t0", "t1", "ev0", "ev1", "tid")

    def __init__(self, name, cat, t0, tid):
        self.name, self.cat, self.t0, self.t1, self.tid = name, cat, t0, t0, tid
        self.ev0 = self.ev1 = None


class Tracer:
    """Context manager that records native calls while it is active.

    ``device_time`` records two CUDA events per call (adds about 4 us of host time per call);
    the device durations are resolved by :meth:`finish`, which synchronises once.
    """

    def __init__(self, device_time: bool = False, nvtx: bool = False, max_spans: int = 1 << 20):
        self.device_time, self.nvtx, self.max_spans = device_time, nvtx, max_spans
        self.spans: List[_Span] = []
        self.dropped = 0
        self._origin = time.perf_counter()
        self._open: Dict[int, List[_Span]] = defaultdict(list)
        self._prev = None

    # -- activation ---------------------------------------------------------------------
    def __enter__(self):
        global _active
        self._prev = _active
        _active = self
        _l.set_call_hook(_hooked_call)
        return self

    def __exit__(self, *exc):
        global _active
        _active = self._prev
        if _active is None:
            _l.set_call_hook(None)
        self.finish()
        return False

    # -- recording ----------------------------------------------------------------------
    def begin(self, name: str, cat: str = "kernel") -> Optional[_Span]:
        if len(self.spans) >= self.max_spans:
            self.dropped += 1
            return None
        s = _Span(name, cat, time.perf_counter(), threading.get_ident())
        if self.nvtx and torch.cuda.is_available():
            torch.cuda.nvtx.range_push(name)
        if self.device_time and cat == "kernel" and torch.cuda.is_available():
            s.ev0 = torch.cuda.Event(enable_timing=True)
            s.ev0.record()
        self.spans.append(s)
        return s

    def end(self, s: Optional[_Span]) -> None:
        if s is None:
            return
        if s.ev0 is not None:
            s.ev1 = torch.cuda.Event(enable_timing=True)
            s.ev1.record()
        if self.nvtx and torch.cuda.is_available():
            torch.cuda.nvtx.range_pop()
        s.t1 = time.perf_counter()

    def finish(self) -> None:
        """Resolves device durations (one synchronise)."""
        if any(s.ev1 is not None for s in self.spans):
            torch.cuda.synchronize()

    # -- reports ------------------------------------------------------------------------
    def summary(self) -> List[dict]:
        """One row per name: calls, host microseconds, device milliseconds (if recorded)."""
        rows: Dict[tuple, dict] = {}
        for s in self.spans:
            r = rows.setdefault((s.cat, s.name), dict(name=s.name, cat=s.cat, calls=0, host_us=0.0,
                                                      device_ms=None))
            r["calls"] += 1
            r["host_us"] += (s.t1 - s.t0) * 1e6
            if s.ev1 is not None:
                r["device_ms"] = (r["device_ms"] or 0.0) + s.ev0.elapsed_time(s.ev1)
        key = (lambda r: -(r["device_ms"] or 0.0)) if self.device_time else (lambda r: -r["host_us"])
        return sorted(rows.values(), key=key)

    def table(self) -> str:
        lines = [f"{'name':32s} {'cat':7s} {'calls':>7s} {'host us':>10s} {'device ms':>10s}"]
        for r in self.summary():
            dev = "-" if r["device_ms"] is None else f"{r['device_ms']:.3f}"
            lines.append(f"{r['name'][:32]:32s} {r['cat']:7s} {r['calls']:7d} {r['host_us']:10.1f} {dev:>10s}")
        if self.dropped:
            lines.append(f"({self.dropped} spans dropped: max_spans reached)")
        return "\n".join(lines)

    def chrome_trace(self) -> dict:
        """Trace-event JSON: host spans as complete events ("ph": "X"), one row per thread;
        device durations, when recorded, ride along in ``args``."""
        ev = []
        for s in self.spans:
            e = dict(name=s.name, cat=s.cat, ph="X", pid=0, tid=s.tid % 100000,
                     ts=(s.t0 - self._origin) * 1e6, dur=max((s.t1 - s.t0) * 1e6, 0.001))
            if s.ev1 is not None:
                e["args"] = {"device_ms": s.ev0.elapsed_time(s.ev1)}
            ev.append(e)
        return {"traceEvents": ev, "displayTimeUnit": "ms"}

    def save(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump(self.chrome_trace(), f)


def _hooked_call(name: str, fn, args):
    t = _active
    if t is None:
        return fn(*args)
    s = t.begin(name)
    try:
        return fn(*args)
    finally:
        t.end(s)


def trace_modules(module: torch.nn.Module, tracer: Optional[Tracer] = None):
    """Registers forward pre / post hooks on every sub-module so that module spans (category
    ``module``, named by the module path) enclose the kernel spans.  Returns the handles;
    call ``h.remove()`` on each to detach."""
    handles = []
    for path, m in module.named_modules():
        label = f"{path or 'model'}:{type(m).__name__}"
        stack: List[Optional[_Span]] = []

        def pre(_m, _inp, label=label, stack=stack):
            t = tracer or _active
            stack.append(t.begin(label, "module") if t is not None else None)

        def post(_m, _inp, _out, stack=stack):
            t = tracer or _active
            s = stack.pop() if stack else None
            if t is not None:
                t.end(s)

        handles.append(m.register_forward_pre_hook(pre))
        handles.append(m.register_forward_hook(post))
    return handles


class StepTimer:
    """Per-step device timing.  ``start()`` / ``stop()`` bracket one step with CUDA events on
    the current stream (``perf_counter`` on CPU); ``report()`` synchronises once and returns
    ``{"steps", "mean_ms", "median_ms", "max_ms"}``, each the MAX over ranks when a process
    group is initialised (a multi-GPU step is as slow as its slowest rank)."""

    def __init__(self, device: Optional[torch.device] = None):
        self.cuda = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
        self._pairs = []
        self._t0 = None

    def start(self):
        if self.cuda:
            self._t0 = torch.cuda.Event(enable_timing=True)
            self._t0.record()
        else:
            self._t0 = time.perf_counter()

    def stop(self):
        if self.cuda:
            e1 = torch.cuda.Event(enable_timing=True)
            e1.record()
            self._pairs.append((self._t0, e1))
        else:
            self._pairs.append((self._t0, time.perf_counter()))

    def times_ms(self) -> List[float]:
        if self.cuda:
            torch.cuda.synchronize()
            return [a.elapsed_time(b) for a, b in self._pairs]
        return [(b - a) * 1e3 for a, b in self._pairs]

    def report(self) -> dict:
        import statistics
        ts = self.times_ms()
        if not ts:
            return dict(steps=0, mean_ms=0.0, median_ms=0.0, max_ms=0.0)
        vals = [sum(ts) / len(ts), statistics.median(ts), max(ts)]
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            dev = "cuda" if (self.cuda and dist.get_backend() == "nccl") else "cpu"
            t = torch.tensor(vals, dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            vals = t.tolist()
        return dict(steps=len(ts), mean_ms=vals[0], median_ms=vals[1], max_ms=vals[2])

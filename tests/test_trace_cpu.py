"""Tracer, module spans and the step timer (host-side logic; native calls are faked)."""
import json

import torch

from gonn_b200 import lib as _l
from gonn_b200 import nn
from gonn_b200.utils.trace import StepTimer, Tracer, trace_modules


def _fake_native(monkeypatch, name="gb_fake_kernel", rc=0):
    calls = []

    def fn(*args):
        calls.append(args)
        return rc

    monkeypatch.setitem(_l._fn_cache, name, fn)
    return calls


def test_tracer_records_native_calls(monkeypatch, tmp_path):
    calls = _fake_native(monkeypatch)
    _l.call("gb_fake_kernel", 1, 2)          # before: no tracer, no record
    with Tracer() as tr:
        for _ in range(3):
            _l.call("gb_fake_kernel", 7)
    _l.call("gb_fake_kernel")                # after: hook removed
    assert len(calls) == 5 and _l._call_hook is None
    rows = tr.summary()
    assert rows == [dict(name="gb_fake_kernel", cat="kernel", calls=3, host_us=rows[0]["host_us"],
                         device_ms=None)]
    assert "gb_fake_kernel" in tr.table()
    path = tmp_path / "trace.json"
    tr.save(str(path))
    ev = json.loads(path.read_text())["traceEvents"]
    assert len(ev) == 3 and all(e["ph"] == "X" and e["dur"] > 0 for e in ev)


def test_tracer_propagates_errors_and_nests(monkeypatch):
    _fake_native(monkeypatch)
    with Tracer() as outer:
        with Tracer() as inner:
            _l.call("gb_fake_kernel")
        assert _l._call_hook is not None      # the outer tracer is active again
        _l.call("gb_fake_kernel")
    assert len(inner.spans) == 1 and len(outer.spans) == 1

    def boom(*a):
        raise ValueError("x")

    monkeypatch.setitem(_l._fn_cache, "gb_boom", boom)
    with Tracer() as tr:
        try:
            _l.call("gb_boom")
        except ValueError:
            pass
    assert tr.spans[0].t1 >= tr.spans[0].t0 and _l._call_hook is None


def test_span_limit(monkeypatch):
    _fake_native(monkeypatch)
    with Tracer(max_spans=2) as tr:
        for _ in range(5):
            _l.call("gb_fake_kernel")
    assert len(tr.spans) == 2 and tr.dropped == 3 and "dropped" in tr.table()


def test_module_spans_enclose_kernels(monkeypatch):
    _fake_native(monkeypatch)

    class Leaf(torch.nn.Module):
        def forward(self, x):
            _l.call("gb_fake_kernel")
            return x + 1

    model = nn.Sequential(Leaf(), Leaf())
    with Tracer() as tr:
        handles = trace_modules(model)
        model(torch.zeros(2))
        for h in handles:
            h.remove()
        model(torch.zeros(2))                 # detached: only kernel spans
    mods = [s for s in tr.spans if s.cat == "module"]
    kers = [s for s in tr.spans if s.cat == "kernel"]
    assert [m.name for m in mods] == ["model:Sequential", "0:Leaf", "1:Leaf"]
    assert len(kers) == 4
    assert mods[1].t0 <= kers[0].t0 and kers[0].t1 <= mods[1].t1 <= mods[0].t1


def test_step_timer_cpu():
    st = StepTimer(device="cpu")
    for _ in range(4):
        st.start()
        torch.randn(64, 64) @ torch.randn(64, 64)
        st.stop()
    r = st.report()
    assert r["steps"] == 4 and 0 < r["median_ms"] <= r["max_ms"] and r["mean_ms"] <= r["max_ms"]
    assert StepTimer(device="cpu").report()["steps"] == 0

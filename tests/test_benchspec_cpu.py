"""Cross-framework benchmark specification: record schema, validation, aggregation."""
import json

import pytest

from gonn_b200.utils import benchspec as bs


def test_run_emits_the_specified_records(tmp_path):
    small = dict(matmul_sizes=(16, 32), vector_sizes=(1000,), iters={"matmul": 3, "elementwise_add": 3, "relu": 3})
    for fw in ("gonn_b200", "pytorch"):
        recs = bs.run(fw, "cpu", dtypes=("float32", "float64"), **small)
        assert len(recs) == 2 * (2 + 2)
        for r in recs:
            assert set(r) == set(bs.REQUIRED) | {"gflops"}
            assert r["transfer"] == "host" and r["ms_per_iter"] > 0 and r["iters"] == 3
            assert (r["gflops"] is not None) == (r["op"] == "matmul")
        path = bs.write(recs, str(tmp_path))
        assert path.endswith(f"{fw}_cpu.json") and isinstance(json.load(open(path)), list)
    md = bs.aggregate(bs.load(str(tmp_path)))
    assert "## matmul - throughput (GFLOP/s, higher is better)" in md
    assert "| gonn_b200 (cpu) |" in md and "| pytorch (cpu) |" in md
    assert "| framework / device | N=16 | N=32 |" in md and "M=1,000" in md
    assert "* gonn_b200 (cpu): `host`" in md


def test_validate_rejects_incomplete_records():
    good = dict(framework="x", device="cpu", dtype="float64", op="relu", size=1, ms_per_iter=1.0,
                gflops=None, iters=1, transfer="host")
    bs.validate([good])
    with pytest.raises(ValueError):
        bs.validate([{k: v for k, v in good.items() if k != "transfer"}])
    with pytest.raises(ValueError):
        bs.validate([dict(good, op="matmul")])


def test_aggregate_fills_missing_cells():
    recs = [dict(framework="a", device="cpu", dtype="float64", op="matmul", size=8, ms_per_iter=1.0,
                 gflops=2.0, iters=1, transfer="host"),
            dict(framework="b", device="cuda", dtype="float64", op="matmul", size=16, ms_per_iter=2.0,
                 gflops=4.0, iters=1, transfer="device-resident")]
    md = bs.aggregate(recs)
    assert "| a (cpu) | 2.0 | - |" in md and "| b (cuda) | - | 4.0 |" in md

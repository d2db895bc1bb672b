"""The reference's cross-framework benchmark specification, runner and aggregator.

The specification (benchmark/BENCH_SPEC.md of the reference): ``matmul`` (square, N in 256,
512, 1024, 2048; GFLOP/s = 2 N^3 / time), ``elementwise_add`` and ``relu`` (length 1e6 and
1e7), float32 and float64, 5 warm-up iterations, the MEDIAN of 20 (matmul) or 50
(elementwise) timed iterations with a device synchronise inside every timed iteration, and
one JSON array per (framework, device) of records

    {"framework", "device", "dtype", "op", "size", "ms_per_iter", "gflops", "iters", "transfer"}

where ``transfer`` says what was timed: ``host`` on CPU, ``device-resident`` when operands
already live on the GPU.  bfloat16 is added as a third dtype on CUDA (the tensor-core path).

    python -m gonn_b200.utils.benchspec run --device cuda --out results/
    python -m gonn_b200.utils.benchspec aggregate results/ > RESULTS.md

``run`` writes ``gonn_b200_<device>.json`` and ``pytorch_<device>.json`` (the same ops
through stock torch, for the side-by-side table the reference publishes in
benchmark/RESULTS.md).
"""
from __future__ import annotations

import glob
import json
import os
import statistics
import sys
import time
from typing import Callable, Dict, Iterable, List, Optional, Sequence

import torch

MATMUL_SIZES = (256, 512, 1024, 2048)
VECTOR_SIZES = (1_000_000, 10_000_000)
WARMUP = 5
ITERS = {"matmul": 20, "elementwise_add": 50, "relu": 50}
REQUIRED = ("framework", "device", "dtype", "op", "size", "ms_per_iter", "iters", "transfer")
_DTYPES = {"float32": torch.float32, "float64": torch.float64, "bfloat16": torch.bfloat16}


def _median_ms(fn: Callable[[], object], iters: int, cuda: bool) -> float:
    for _ in range(WARMUP):
        fn()
    if cuda:
        torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        t0 = time.perf_counter()
        fn()
        if cuda:
            torch.cuda.synchronize()     # inside the timed iteration, as the specification asks
        ts.append((time.perf_counter() - t0) * 1e3)
    return statistics.median(ts)


def _ops(framework: str) -> Dict[str, Callable]:
    if framework == "pytorch":
        return {"matmul": torch.matmul, "elementwise_add": torch.add, "relu": torch.relu}
    from .. import tensor as T
    return {"matmul": T.MatMul, "elementwise_add": T.Add, "relu": lambda x: T.Unary(x, "relu")}


def run(framework: str = "gonn_b200", device: str = "cpu", dtypes: Optional[Sequence[str]] = None,
        matmul_sizes: Iterable[int] = MATMUL_SIZES, vector_sizes: Iterable[int] = VECTOR_SIZES,
        iters: Optional[Dict[str, int]] = None) -> List[dict]:
    """Runs the specification for one framework on one device and returns the records."""
    cuda = device == "cuda"
    if dtypes is None:
        dtypes = ("float32", "float64") + (("bfloat16",) if cuda else ())
    iters = {**ITERS, **(iters or {})}
    ops = _ops(framework)
    transfer = "device-resident" if cuda else "host"
    gen = torch.Generator(device="cpu").manual_seed(0)
    out: List[dict] = []

    def rec(op, dt, size, ms, flops=None):
        out.append(dict(framework=framework, device=device, dtype=dt, op=op, size=size, ms_per_iter=ms,
                        gflops=(flops / 1e9 / (ms / 1e3)) if flops else None, iters=iters[op],
                        transfer=transfer))

    with torch.no_grad():
        for dt in dtypes:
            td = _DTYPES[dt]
            for n in matmul_sizes:
                a = torch.randn(n, n, generator=gen).to(device=device, dtype=td)
                b = torch.randn(n, n, generator=gen).to(device=device, dtype=td)
                rec("matmul", dt, n, _median_ms(lambda: ops["matmul"](a, b), iters["matmul"], cuda),
                    2.0 * n ** 3)
            for m in vector_sizes:
                x = torch.randn(m, generator=gen).to(device=device, dtype=td)
                y = torch.randn(m, generator=gen).to(device=device, dtype=td)
                rec("elementwise_add", dt, m,
                    _median_ms(lambda: ops["elementwise_add"](x, y), iters["elementwise_add"], cuda))
                rec("relu", dt, m, _median_ms(lambda: ops["relu"](x), iters["relu"], cuda))
    return out


def validate(records: Iterable[dict]) -> None:
    """Raises ``ValueError`` if a record misses a required key or a matmul record has no
    ``gflops`` (the two rules of the specification's output format)."""
    for r in records:
        miss = [k for k in REQUIRED if k not in r]
        if miss:
            raise ValueError(f"record {r} misses {miss}")
        if r["op"] == "matmul" and r.get("gflops") is None:
            raise ValueError(f"matmul record without gflops: {r}")


def write(records: List[dict], out_dir: str) -> str:
    validate(records)
    os.makedirs(out_dir, exist_ok=True)
    path = os.path.join(out_dir, f"{records[0]['framework']}_{records[0]['device']}.json")
    with open(path, "w") as f:
        json.dump(records, f, indent=1)
    return path


# -- aggregation ------------------------------------------------------------------------

def load(results_dir: str) -> List[dict]:
    recs: List[dict] = []
    for p in sorted(glob.glob(os.path.join(results_dir, "*.json"))):
        with open(p) as f:
            data = json.load(f)
        if isinstance(data, list):
            recs.extend(r for r in data if isinstance(r, dict) and "op" in r)
    validate(recs)
    return recs


def _table(recs: List[dict], op: str, dtype: str, field: str, size_label: str, fmt: str) -> List[str]:
    rows = [r for r in recs if r["op"] == op and r["dtype"] == dtype and r.get(field) is not None]
    if not rows:
        return []
    sizes = sorted({r["size"] for r in rows})
    who = sorted({(r["framework"], r["device"]) for r in rows})
    lines = [f"### {dtype}", "",
             "| framework / device | " + " | ".join(f"{size_label}={s:,}" for s in sizes) + " |",
             "|---|" + "---|" * len(sizes)]
    for fw, dev in who:
        cells = []
        for s in sizes:
            v = [r[field] for r in rows if (r["framework"], r["device"], r["size"]) == (fw, dev, s)]
            cells.append(format(v[-1], fmt) if v else "-")
        lines.append(f"| {fw} ({dev}) | " + " | ".join(cells) + " |")
    return lines + [""]


def aggregate(recs: List[dict]) -> str:
    """Markdown report in the layout of the reference's generated results file: matmul
    throughput, matmul latency, then add and relu latency, one table per dtype."""
    dts = [d for d in ("float64", "float32", "bfloat16") if any(r["dtype"] == d for r in recs)]
    fws = sorted({r["framework"] for r in recs})
    out = ["# Cross-framework benchmark results", "",
           "Generated by `python -m gonn_b200.utils.benchspec aggregate`; medians, methodology in the "
           "module's docstring.", "", "Frameworks present: " + ", ".join(fws) + ".", ""]
    sections = [("matmul - throughput (GFLOP/s, higher is better)", "matmul", "gflops", "N", ".1f"),
                ("matmul - latency (ms/iter, lower is better)", "matmul", "ms_per_iter", "N", ".3f"),
                ("elementwise add - latency (ms/iter, lower is better)", "elementwise_add", "ms_per_iter", "M", ".3f"),
                ("relu - latency (ms/iter, lower is better)", "relu", "ms_per_iter", "M", ".3f")]
    for title, op, field, lab, fmt in sections:
        body: List[str] = []
        for dt in dts:
            body += _table(recs, op, dt, field, lab, fmt)
        if body:
            out += [f"## {title}", ""] + body
    labels = sorted({(r["framework"], r["device"], r["transfer"]) for r in recs})
    out += ["## What was timed", ""] + [f"* {fw} ({dev}): `{tr}`" for fw, dev, tr in labels] + [""]
    return "\n".join(out)


def main(argv: List[str]) -> None:
    if not argv or argv[0] not in ("run", "aggregate"):
        raise SystemExit(__doc__)
    if argv[0] == "aggregate":
        print(aggregate(load(argv[1] if len(argv) > 1 else "results")))
        return
    import argparse
    ap = argparse.ArgumentParser(prog="benchspec run")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--out", default="results")
    ap.add_argument("--frameworks", default="gonn_b200,pytorch")
    ap.add_argument("--dtypes", default=None, help="comma-separated subset of float32,float64,bfloat16")
    a = ap.parse_args(argv[1:])
    for fw in a.frameworks.split(","):
        recs = run(fw, a.device, a.dtypes.split(",") if a.dtypes else None)
        print(write(recs, a.out), file=sys.stderr)
        for r in recs:
            print(json.dumps(r), flush=True)


if __name__ == "__main__":
    main(sys.argv[1:])

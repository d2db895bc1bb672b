"""Kernel-level benchmark configs of ``bench.py`` (``--config gemm | flash | add``), both arms.

Both arms run the same shapes with the same FLOP conventions (matmul ``2 m k n``; attention
``4 BH S^2 d``, halved when causal: benchmark/BENCH_SPEC.md:11, benchmark/flashattn/main.go:138-142)
and the same protocol as the reference's in-library loops (backend/cuda/gonn_cuda.cu:255-294,
532-592, 673-690): operands allocated once on the device, five or more untimed calls, then
``iters`` back-to-back calls between two CUDA events.  The headline shape of every config has
operands larger than the 126 MB L2, so back-to-back calls still stream from HBM.

* reference arm: only ``baseline/reference_lib.py`` (the reference's library through ctypes);
  nothing of ``gonn_b200`` is imported.
* own arm: ``gonn_b200.cuda`` (``BenchMatMulF16Dev``, ``BenchMatMulDev``, ``BenchFlashAttn``,
  ``BenchAddDev``, ``FlashAttnFwd`` / ``FlashAttnBwd``) and ``gonn_b200.backend``.

The end-to-end value of each config goes through the call a user makes with host data:
upload from (pinned) host memory, the operator, download of the result, every iteration.
"""
from __future__ import annotations

import math
import os
import statistics
import subprocess
import threading
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
          "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
          "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

# published by the reference on its own GPU (RTX 3060): benchmark/REPORT.md:164,
# benchmark/RESULTS.md:88, benchmark/REPORT.md:24
PUBLISHED = {"gemm": ("fp16 N=2048", 24.464, "TFLOP/s"),
             "flash": ("fp64 (16,2048,64) causal fwd", 0.0866, "TFLOP/s"),
             "add": ("fp32 n=1e7", 3 * 1e7 * 4 / 0.369e-3 / 1e9, "GB/s")}


class Clocks:
    """Samples ``nvidia-smi`` (read-only) every 200 ms between ``start`` and ``stop``."""

    def __init__(self, gpu: int = 0):
        self.gpu, self.rows, self.proc, self.th = gpu, [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={_QUERY}", "--format=csv,noheader,nounits", "-i", str(self.gpu),
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return self
        self.th = threading.Thread(target=self._read, daemon=True)
        self.th.start()
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 9:
                self.rows.append(parts)

    def stop(self) -> dict:
        if self.proc is not None:
            time.sleep(0.25)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            if self.th is not None:
                self.th.join(timeout=2)
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def loaded_repo_libraries() -> list:
    """Shared objects under the repository that are mapped into this process."""
    libs = set()
    try:
        with open("/proc/self/maps") as f:
            for line in f:
                path = line.rstrip("\n").split(" ")[-1]
                if path.endswith(".so") and os.path.realpath(path).startswith(os.path.realpath(ROOT)):
                    libs.add(os.path.relpath(os.path.realpath(path), os.path.realpath(ROOT)))
    except OSError:
        pass
    return sorted(libs)


def _gemm_tf(n, ms):
    return 2.0 * n ** 3 / ms / 1e9


def _attn_tf(BH, S, d, causal, ms):
    return 4.0 * BH * S * S * d * (0.5 if causal else 1.0) / ms / 1e9


REF_ATTN_SHAPES = ((16, 2048, 64), (32, 1024, 64), (64, 512, 64))   # benchmark/flashattn/main.go:127-132
CONFIG4 = (8 * 16, 4096, 128)                                          # B=8, H=16, S=4096, head_dim 128


def _pinned(shape, seed):
    import torch
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, dtype=torch.float64, generator=g).pin_memory()


# ---------------------------------------------------------------------------------------------
# reference arm
# ---------------------------------------------------------------------------------------------

def run_reference(config: str, steps: int, warmup: int, quick: bool) -> dict:
    import numpy as np
    from . import reference_lib as R
    if R.build() is None:
        return {"impl": "reference", "unavailable": "baseline/_ref/libgonn_cuda.so is absent and the reference "
                                                    "source tree is not present to build it"}
    ref = R.load()
    iters = max(1, steps)
    sweep, e2e, notes = [], None, {}
    clocks = Clocks(0).start()
    if config == "gemm":
        n0 = 8192
        ms = ref.gonn_bench_matmul_f16_dev(n0, n0, n0, iters)
        clk = clocks.stop()
        value, unit, msps = _gemm_tf(n0, ms), "TFLOP/s", ms
        dtype, shape = "fp16 (fp32 accumulate, cublasGemmEx)", f"{n0}x{n0}x{n0}"
        if not quick:
            for n in (2048, 4096):
                t = ref.gonn_bench_matmul_f16_dev(n, n, n, iters)
                sweep.append({"op": "matmul", "dtype": "fp16", "n": n, "ms": t, "tflops": _gemm_tf(n, t)})
            for f32, name in ((1, "fp32"), (0, "fp64")):
                for n in (2048, 4096):
                    t = ref.gonn_bench_matmul_dev(n, n, n, iters, f32)
                    sweep.append({"op": "matmul", "dtype": name, "n": n, "ms": t, "tflops": _gemm_tf(n, t)})
        n = 2048
        a, b = _pinned((n, n), 1).numpy(), _pinned((n, n), 2).numpy()
        c = np.empty((n, n), dtype=np.float64)
        call = lambda: ref.gonn_gemm(R.dptr(a), R.dptr(b), R.dptr(c), 1, n, n, n, 0, 0)
        for _ in range(max(3, warmup)):
            call()
        t0 = time.perf_counter()
        for _ in range(iters):
            rc = call()
        dt = (time.perf_counter() - t0) / iters
        assert rc == 0, rc
        e2e = {"value": 2.0 * n ** 3 / dt / 1e12, "unit": "TFLOP/s", "what": f"gonn_gemm fp64 {n}^3 on host arrays "
               "(upload, cublasDgemm, download every call), wall clock", "ms_per_step": dt * 1e3,
               "h2d_bytes_per_step": 2 * n * n * 8, "d2h_bytes_per_step": n * n * 8,
               "checksum": float(c[0, 0])}
    elif config == "flash":
        BH, S, d = CONFIG4
        it4 = min(iters, 2)                      # seconds per call at this shape: fewer timed calls
        ms = ref.gonn_bench_flash_attn_f64(BH, S, d, it4, 1)
        clk = clocks.stop()
        value, unit, msps = _attn_tf(BH, S, d, True, ms), "TFLOP/s", ms
        dtype, shape = "fp64 (the reference's only attention kernel)", f"BH={BH} S={S} d={d} causal, forward"
        notes["timed_iters"] = it4
        for bh, s, dd in REF_ATTN_SHAPES if not quick else REF_ATTN_SHAPES[:1]:
            for causal in (0, 1):
                t = ref.gonn_bench_flash_attn_f64(bh, s, dd, iters, causal)
                sweep.append({"op": "attention_fwd", "dtype": "fp64", "BH": bh, "S": s, "d": dd, "causal": bool(causal),
                              "ms": t, "tflops": _attn_tf(bh, s, dd, causal, t)})
        # end to end: forward + backward through the host-pointer entry points
        bh, s, dd = REF_ATTN_SHAPES[0]
        q, k, v, do = (_pinned((bh, s, dd), 10 + i).numpy() for i in range(4))
        o, dq, dk, dv = (np.empty_like(q) for _ in range(4))
        L = np.empty((bh, s), dtype=np.float64)
        scale = 1.0 / math.sqrt(dd)

        def fwd_bwd():
            ref.gonn_flash_attn_f64_fwd(R.dptr(q), R.dptr(k), R.dptr(v), R.dptr(o), R.dptr(L), bh, s, dd, scale, 1)
            ref.gonn_flash_attn_f64_bwd(R.dptr(q), R.dptr(k), R.dptr(v), R.dptr(o), R.dptr(L), R.dptr(do),
                                        R.dptr(dq), R.dptr(dk), R.dptr(dv), bh, s, dd, scale, 1)
        fwd_bwd()
        t0 = time.perf_counter()
        n_e2e = min(iters, 3)
        for _ in range(n_e2e):
            fwd_bwd()
        dt = (time.perf_counter() - t0) / n_e2e
        fl = 3.5 * 4.0 * bh * s * s * dd * 0.5
        e2e = {"value": fl / dt / 1e12, "unit": "TFLOP/s", "what": f"gonn_flash_attn_f64_fwd + _bwd on host arrays, "
               f"(BH,S,d)=({bh},{s},{dd}) causal, forward + backward = 3.5 x forward FLOPs, wall clock",
               "ms_per_step": dt * 1e3, "h2d_bytes_per_step": (3 + 6) * q.nbytes + L.nbytes,
               "d2h_bytes_per_step": 4 * q.nbytes + L.nbytes, "checksum": float(dq[0, 0, 0])}
        # the backward at the headline shape is reached only through the host-pointer call; its
        # kernel serialises on float64 atomics, so it runs only when the small shape predicts < 90 s
        bwd_small = dt
        pred = bwd_small * (BH / bh) * (S / s) ** 2 * (d / dd) * 1.5
        notes["bwd_config4_predicted_s"] = pred
        if not quick and pred < 90.0:
            sh = (BH, S, d)
            q, k, v, do = (_pinned(sh, 20 + i).numpy() for i in range(4))
            o, dq, dk, dv = (np.empty_like(q) for _ in range(4))
            L = np.empty((BH, S), dtype=np.float64)
            sc = 1.0 / math.sqrt(d)
            ref.gonn_flash_attn_f64_fwd(R.dptr(q), R.dptr(k), R.dptr(v), R.dptr(o), R.dptr(L), BH, S, d, sc, 1)
            t0 = time.perf_counter()
            ref.gonn_flash_attn_f64_bwd(R.dptr(q), R.dptr(k), R.dptr(v), R.dptr(o), R.dptr(L), R.dptr(do),
                                        R.dptr(dq), R.dptr(dk), R.dptr(dv), BH, S, d, sc, 1)
            tb = time.perf_counter() - t0
            sweep.append({"op": "attention_bwd", "dtype": "fp64", "BH": BH, "S": S, "d": d, "causal": True,
                          "ms": tb * 1e3, "tflops": 2.5 * _attn_tf(BH, S, d, True, tb * 1e3),
                          "timing": "one host-pointer call, wall clock, includes 9 uploads and 3 downloads of 537 MB"})
    else:  # add
        n0 = 10 ** 8
        ms = ref.gonn_bench_add_dev(n0, iters, 1)
        clk = clocks.stop()
        value, unit, msps = 3.0 * n0 * 4 / ms / 1e6, "GB/s", ms
        dtype, shape = "fp32", f"n={n0}"
        if not quick:
            for f32, name, esz in ((1, "fp32", 4), (0, "fp64", 8)):
                for n in (10 ** 6, 10 ** 7):
                    t = ref.gonn_bench_add_dev(n, iters, f32)
                    sweep.append({"op": "add", "dtype": name, "n": n, "ms": t, "gbs": 3.0 * n * esz / t / 1e6})
        n = 10 ** 7
        a, b = _pinned((n,), 3).numpy(), _pinned((n,), 4).numpy()
        c = np.empty(n, dtype=np.float64)
        call = lambda: ref.gonn_binary(0, R.dptr(a), R.dptr(b), R.dptr(c), n)
        for _ in range(max(3, warmup)):
            call()
        t0 = time.perf_counter()
        for _ in range(iters):
            rc = call()
        dt = (time.perf_counter() - t0) / iters
        assert rc == 0, rc
        e2e = {"value": 3.0 * n * 8 / dt / 1e9, "unit": "GB/s", "what": f"gonn_binary(add) fp64 n={n} on host arrays "
               "(upload, kernel, download every call), wall clock", "ms_per_step": dt * 1e3,
               "h2d_bytes_per_step": 2 * n * 8, "d2h_bytes_per_step": n * 8, "checksum": float(c[0])}
    if msps < 0:
        return {"impl": "reference", "unavailable": "the reference's benchmark loop returned -1 (cudaMalloc failed)"}
    return _line("reference", config, value, unit, msps, dtype, shape, steps, max(5, warmup), clk, e2e, sweep, 0, notes)


# ---------------------------------------------------------------------------------------------
# this framework's arm
# ---------------------------------------------------------------------------------------------

def run_ours(config: str, steps: int, warmup: int, quick: bool) -> dict:
    import torch
    from gonn_b200 import backend as gb
    from gonn_b200 import cuda as C
    from gonn_b200 import lib as gl
    from gonn_b200.ops import attention as A
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    iters = max(1, steps)
    sweep, e2e, notes = [], None, {}
    be = gb.NewCUDA()
    clocks = Clocks(0).start()
    if config == "gemm":
        n0 = 8192
        C.BenchMatMulF16Dev(n0, n0, n0, max(0, warmup - 5) + 1)          # extra warm-up beyond the loop's own five
        k0 = gl.kernel_count
        ms = C.BenchMatMulF16Dev(n0, n0, n0, iters)
        launches = gl.kernel_count - k0 - 5
        clk = clocks.stop()
        value, unit, msps = _gemm_tf(n0, ms), "TFLOP/s", ms
        dtype, shape = "fp16 (fp32 accumulate, tcgen05)", f"{n0}x{n0}x{n0}"
        if not quick:
            for n in (2048, 4096):
                t = C.BenchMatMulF16Dev(n, n, n, iters)
                sweep.append({"op": "matmul", "dtype": "fp16", "n": n, "ms": t, "tflops": _gemm_tf(n, t)})
                t = C.BenchMatMulF16Dev(n, n, n, iters, dtype=torch.bfloat16)
                sweep.append({"op": "matmul", "dtype": "bf16", "n": n, "ms": t, "tflops": _gemm_tf(n, t)})
            for f32, name in ((True, "fp32"), (False, "fp64")):
                for n in (2048, 4096):
                    t = C.BenchMatMulDev(n, n, n, iters, f32)
                    sweep.append({"op": "matmul", "dtype": name, "n": n, "ms": t, "tflops": _gemm_tf(n, t)})
        n = 2048
        a, b = _pinned((n, n), 1), _pinned((n, n), 2)
        c = torch.empty(n, n, dtype=torch.float64).pin_memory()

        def call():
            out = be.Gemm(a.to(dev, non_blocking=True), b.to(dev, non_blocking=True), 1, n, n, n)
            c.copy_(out.view(n, n))          # device -> host; synchronises

        for _ in range(max(3, warmup)):
            call()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(iters):
            call()
        torch.cuda.synchronize()
        dt = (time.perf_counter() - t0) / iters
        e2e = {"value": 2.0 * n ** 3 / dt / 1e12, "unit": "TFLOP/s", "what": f"backend.Gemm fp64 {n}^3 from pinned host "
               "arrays (upload, kernel, download every call), wall clock", "ms_per_step": dt * 1e3,
               "h2d_bytes_per_step": 2 * n * n * 8, "d2h_bytes_per_step": n * n * 8, "checksum": float(c[0, 0])}
    elif config == "flash":
        BH, S, d = CONFIG4
        C.BenchFlashAttn(BH, S, d, max(1, warmup - 5), True)
        k0 = gl.kernel_count
        ms = C.BenchFlashAttn(BH, S, d, iters, True)
        launches = gl.kernel_count - k0 - 5
        clk = clocks.stop()
        value, unit, msps = _attn_tf(BH, S, d, True, ms), "TFLOP/s", ms
        dtype, shape = "bf16 (fp32 accumulate, tcgen05)", f"BH={BH} S={S} d={d} causal, forward"
        for bh, s, dd in REF_ATTN_SHAPES if not quick else REF_ATTN_SHAPES[:1]:
            for causal in (False, True):
                t = C.BenchFlashAttn(bh, s, dd, iters, causal)
                sweep.append({"op": "attention_fwd", "dtype": "bf16", "BH": bh, "S": s, "d": dd, "causal": causal,
                              "ms": t, "tflops": _attn_tf(bh, s, dd, causal, t)})
                if not quick:
                    t = C.BenchFlashAttn(bh, s, dd, iters, causal, dtype=torch.float64)
                    sweep.append({"op": "attention_fwd", "dtype": "fp64", "BH": bh, "S": s, "d": dd, "causal": causal,
                                  "ms": t, "tflops": _attn_tf(bh, s, dd, causal, t)})
        # backward at the headline shape, resident
        q, k, v, do = (torch.randn(1, S, BH, d, device=dev, dtype=torch.bfloat16) for _ in range(4))
        sc = 1.0 / math.sqrt(d)
        o, lse = A.flash_fwd(q, k, v, True, sc)
        tb = C._time_ms(lambda: A.flash_bwd(q, k, v, o, do, lse, True, sc), iters, dev)
        sweep.append({"op": "attention_bwd", "dtype": "bf16", "BH": BH, "S": S, "d": d, "causal": True, "ms": tb,
                      "tflops": 2.5 * _attn_tf(BH, S, d, True, tb), "timing": "resident, CUDA events"})
        del q, k, v, do, o, lse
        bh, s, dd = REF_ATTN_SHAPES[0]
        hq, hk, hv, hdo = (_pinned((bh, s, dd), 10 + i) for i in range(4))
        outs = [torch.empty(bh, s, dd, dtype=torch.float64).pin_memory() for _ in range(4)]
        hl = torch.empty(bh, s, dtype=torch.float64).pin_memory()

        def fwd_bwd():
            o, L = C.FlashAttnFwd(hq, hk, hv, bh, s, dd, None, True, device=dev)
            dq, dk, dv = C.FlashAttnBwd(hq, hk, hv, o, L, hdo, bh, s, dd, None, True, device=dev)
            for dst, src in zip(outs, (o, dq, dk, dv)):
                dst.copy_(src)
            hl.copy_(L)

        fwd_bwd()
        torch.cuda.synchronize()
        n_e2e = min(iters, 3)
        t0 = time.perf_counter()
        for _ in range(n_e2e):
            fwd_bwd()
        torch.cuda.synchronize()
        dt = (time.perf_counter() - t0) / n_e2e
        fl = 3.5 * 4.0 * bh * s * s * dd * 0.5
        nb = hq.numel() * 8
        e2e = {"value": fl / dt / 1e12, "unit": "TFLOP/s", "what": f"cuda.FlashAttnFwd + FlashAttnBwd from pinned host "
               f"float64 arrays, (BH,S,d)=({bh},{s},{dd}) causal, computed in bf16 on the device, forward + backward = "
               "3.5 x forward FLOPs, wall clock", "ms_per_step": dt * 1e3, "h2d_bytes_per_step": 7 * nb,
               "d2h_bytes_per_step": 4 * nb + hl.numel() * 8, "checksum": float(outs[1][0, 0, 0])}
    else:
        n0 = 10 ** 8
        C.BenchAddDev(n0, max(1, warmup - 5), True)
        k0 = gl.kernel_count
        ms = C.BenchAddDev(n0, iters, True)
        launches = gl.kernel_count - k0 - 5
        clk = clocks.stop()
        value, unit, msps = 3.0 * n0 * 4 / ms / 1e6, "GB/s", ms
        dtype, shape = "fp32", f"n={n0}"
        if not quick:
            for f32, name, esz in ((True, "fp32", 4), (False, "fp64", 8)):
                for n in (10 ** 6, 10 ** 7):
                    t = C.BenchAddDev(n, iters, f32)
                    sweep.append({"op": "add", "dtype": name, "n": n, "ms": t, "gbs": 3.0 * n * esz / t / 1e6})
        n = 10 ** 7
        a, b = _pinned((n,), 3), _pinned((n,), 4)
        c = torch.empty(n, dtype=torch.float64).pin_memory()

        def call():
            c.copy_(be.Binary(gb.BinaryKind.Add, a.to(dev, non_blocking=True), b.to(dev, non_blocking=True)))

        for _ in range(max(3, warmup)):
            call()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(iters):
            call()
        torch.cuda.synchronize()
        dt = (time.perf_counter() - t0) / iters
        e2e = {"value": 3.0 * n * 8 / dt / 1e9, "unit": "GB/s", "what": f"backend.Binary(Add) fp64 n={n} from pinned host "
               "arrays (upload, kernel, download every call), wall clock", "ms_per_step": dt * 1e3,
               "h2d_bytes_per_step": 2 * n * 8, "d2h_bytes_per_step": n * 8, "checksum": float(c[0])}
    gl.assert_status_ok()
    return _line("ours", config, value, unit, msps, dtype, shape, steps, max(5, warmup), clk, e2e, sweep, launches, notes)


def _line(impl, config, value, unit, ms, dtype, shape, steps, warmup, clk, e2e, sweep, launches, notes):
    name, pub, pub_unit = PUBLISHED[config]
    metric = {"gemm": "matmul throughput (2mkn FLOPs, resident operands, CUDA events)",
              "flash": "attention forward throughput (4 BH S^2 d FLOPs, halved when causal; resident, CUDA events)",
              "add": "elementwise add bandwidth (3 n elements moved, resident, CUDA events)"}[config]
    out = {"metric": metric, "value": value, "unit": unit, "n_gpus": 1, "steps": steps, "warmup": warmup,
           "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": value / pub,
           "vs_baseline_note": f"published on the reference's own GPU (RTX 3060) for {name}: {pub:.4g} {pub_unit}; "
                               "the value here is for the headline shape in config",
           "dtype": dtype, "data": "synthetic", "impl": impl,
           "config": {"model": f"kernel:{config}", "shape": shape, "global_batch": 1, "seq_len": 0, "parallelism": "single GPU",
                      "cache": "operands of the headline shape exceed the 126 MB L2; back-to-back calls, no explicit flush "
                               "(the protocol of the reference's in-library loops)"},
           "clocks": clk, "e2e": e2e, "gpu_launches": launches, "sweep": sweep,
           "native_so_loaded": loaded_repo_libraries()}
    out.update(notes)
    return out

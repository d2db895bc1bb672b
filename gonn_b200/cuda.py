"""Device-resident buffer API, flash-attention entry points and in-library benchmarks.

The counterpart of the reference's ``backend/cuda`` package (backend/cuda/cuda.go:104-288):

* ``DeviceBuffer`` / ``DevAlloc`` / ``DevUpload`` / ``Download`` / ``Free`` / ``DevSync`` and
  the resident operations ``DevMatMul`` / ``DevAdd`` / ``DevReLU`` (cuda.go:196-243): data is
  uploaded once, kernels run on buffers that stay on the GPU, only results are read back.
  The reference pays two uploads and one download per eager op and added this API to show the
  difference; here every tensor op is resident, so the API is a thin, explicit form of it.
* ``DeviceBufferF16`` / ``DevUploadF16`` / ``DevMatMulF16`` (cuda.go:245-283): 16-bit storage
  with fp32 accumulation.  The reference calls cublasGemmEx; here the product runs on the
  tcgen05 GEMM, in fp16 (as there) or bf16.
* ``FlashAttn`` / ``FlashAttnFwd`` / ``FlashAttnBwd`` over flat ``(BH, S, d)`` arrays
  (cuda.go:125-184), returning the log-sum-exp ``L = m + log(l)`` of the scaled scores from
  the forward and taking it in the backward.
* ``BenchMatMulDev`` / ``BenchAddDev`` / ``BenchMatMulF16Dev`` / ``BenchFlashAttn``
  (cuda.go:104-123, 186-194, 279-282): device-resident loops timed with CUDA events, returning
  milliseconds per iteration.

``Available()`` tells whether a CUDA device and the native library are present;
``Backend()`` returns the backend object to pass to ``gonn_b200.backend.Use``.  Every function
takes an optional ``device`` so that the same calls run on CPU tensors (the oracle path).
"""
from __future__ import annotations

import math
import time
from typing import Optional, Sequence, Tuple

import torch

from . import backend as _backend
from . import lib as _l
from .ops import attention as _attn
from .ops import elementwise as _ew
from .ops.gemm import gemm as _gemm


def Available() -> bool:
    return torch.cuda.is_available() and _l.available()


def Backend() -> "_backend.Backend":
    """The CUDA backend object; raises when no device or no native library is present (the
    reference's stub returns an error from the same call, backend/cuda/cuda_stub.go:16-19)."""
    if not Available():
        raise RuntimeError("cuda.Backend: no CUDA device or native library not built")
    return _backend.NewCUDA()


def _device(device) -> torch.device:
    if device is not None:
        return torch.device(device)
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device: pass device='cpu' to run on the host")
    return torch.device("cuda", torch.cuda.current_device())


class DeviceBuffer:
    """A flat buffer of ``n`` elements that lives on the device until ``Free``."""

    __slots__ = ("t",)

    def __init__(self, t: torch.Tensor):
        self.t = t

    @property
    def n(self) -> int:
        return self.t.numel()

    def Download(self):
        """Copies back to a host float64 array (synchronises)."""
        if self.t is None:
            raise RuntimeError("DeviceBuffer: used after Free")
        return self.t.detach().to("cpu", torch.float64).numpy()

    def Free(self) -> None:
        self.t = None

    def _view(self, *shape):
        if self.t is None:
            raise RuntimeError("DeviceBuffer: used after Free")
        need = math.prod(shape)
        if need > self.t.numel():
            raise ValueError(f"DeviceBuffer of {self.t.numel()} elements used as {shape}")
        return self.t[:need].view(*shape)


class DeviceBufferF16(DeviceBuffer):
    """16-bit storage (fp16 by default, bf16 on request); ``Download`` widens to float64."""


def _alloc(n, dtype, device):
    return torch.zeros(int(n), dtype=dtype, device=_device(device))


def _upload(host, dtype, device):
    h = torch.as_tensor(host, dtype=torch.float64).reshape(-1)
    dev = _device(device)
    if dev.type == "cuda":
        h = h.pin_memory()
    return h.to(dev, dtype=dtype, non_blocking=True)


def DevAlloc(n: int, dtype: torch.dtype = torch.float64, device=None) -> DeviceBuffer:
    return DeviceBuffer(_alloc(n, dtype, device))


def DevUpload(host, dtype: torch.dtype = torch.float64, device=None) -> DeviceBuffer:
    return DeviceBuffer(_upload(host, dtype, device))


def DevAllocF16(n: int, dtype: torch.dtype = torch.float16, device=None) -> DeviceBufferF16:
    return DeviceBufferF16(_alloc(n, dtype, device))


def DevUploadF16(host, dtype: torch.dtype = torch.float16, device=None) -> DeviceBufferF16:
    """Uploads float64 host data and narrows it on the device (the reference converts with a
    kernel after the upload as well, gonn_cuda.cu:633-660)."""
    return DeviceBufferF16(_upload(host, torch.float64, device).to(dtype))


def DevSync() -> None:
    if torch.cuda.is_available():
        torch.cuda.synchronize()


def DevMatMul(a: DeviceBuffer, b: DeviceBuffer, c: DeviceBuffer, m: int, k: int, n: int) -> None:
    """``c (m,n) = a (m,k) @ b (k,n)``, row-major, all three resident."""
    _gemm(a._view(m, k), b._view(k, n), out=c._view(m, n))


def DevMatMulF16(a: DeviceBufferF16, b: DeviceBufferF16, c: DeviceBufferF16, m: int, k: int, n: int) -> None:
    """16-bit operands, fp32 accumulation, 16-bit result (tcgen05 on the device)."""
    _gemm(a._view(m, k), b._view(k, n), out=c._view(m, n))


def DevAdd(a: DeviceBuffer, b: DeviceBuffer, c: DeviceBuffer, n: int) -> None:
    c._view(n).copy_(_ew.binary_forward("add", a._view(n), b._view(n)))


def DevReLU(a: DeviceBuffer, n: int) -> None:
    """In place, as in the reference (cuda.go:242)."""
    v = a._view(n)
    v.copy_(_ew.unary_forward("relu", v))


# -- flash attention over flat (BH, S, d) arrays --------------------------------------------

def _bshd(x, BH: int, S: int, d: int, dtype, device) -> torch.Tensor:
    """(BH, S, d) data as a (1, S, BH, d) view in the kernels' layout (a view when device and
    dtype already match: the head axis gets stride S*d, the sequence axis stride d)."""
    t = x._view(BH, S, d) if isinstance(x, DeviceBuffer) else torch.as_tensor(x).reshape(BH, S, d)
    if t.device != device or t.dtype != dtype:
        t = t.to(device=device, dtype=dtype)
    return t.permute(1, 0, 2).unsqueeze(0)


def _flat(t: torch.Tensor, BH: int, S: int, d: int) -> torch.Tensor:
    return t.squeeze(0).permute(1, 0, 2).contiguous().view(BH, S, d)


def _attn_dtype(dtype, device, d):
    """16-bit tensors of head size 64 / 128 run the tcgen05 kernels; everything else (the
    reference's float64 included) is evaluated in its own precision with tensor ops."""
    if dtype is not None:
        return dtype
    return torch.bfloat16 if (device.type == "cuda" and d % 8 == 0 and 8 <= d <= 128) else torch.float64


def FlashAttnFwd(Q, K, V, BH: int, S: int, d: int, scale: Optional[float] = None, causal: bool = False,
                 dtype: Optional[torch.dtype] = None, device=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns ``(O, L)``: the output ``(BH, S, d)`` and the row log-sum-exp ``(BH, S)`` of the
    scaled (and masked) scores, which the backward needs (cuda.go:141-160)."""
    dev = _device(device)
    dt = _attn_dtype(dtype, dev, d)
    scale = (1.0 / math.sqrt(d)) if scale is None else float(scale)
    q, k, v = (_bshd(x, BH, S, d, dt, dev) for x in (Q, K, V))
    if _attn._kernel_ok(q, k, v):
        o = torch.empty(BH, S, d, dtype=dt, device=dev)       # written in place through a strided view
        _, lse = _attn.flash_fwd(q, k, v, bool(causal), scale, out=o.permute(1, 0, 2).unsqueeze(0))
        return o, lse.view(BH, S)
    if _attn.general_ok(q, k, v):
        # fp32 / fp64 (the reference's kernels are fp64) and odd head sizes: the general fused kernels
        o4, lse = _attn.general_fwd(q, k, v, bool(causal), scale)
        return _flat(o4, BH, S, d), lse.view(BH, S)
    ct = torch.float64 if dt == torch.float64 else torch.float32
    qf, kf, vf = (_flat(t, BH, S, d).to(ct) for t in (q, k, v))
    s = torch.matmul(qf, kf.transpose(1, 2)) * scale
    if causal:
        s = s.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool, device=dev), diagonal=1), -1e30)
    lse = torch.logsumexp(s, dim=-1)
    o = torch.matmul(torch.exp(s - lse.unsqueeze(-1)), vf)
    return o.to(dt), lse


def FlashAttn(Q, K, V, BH: int, S: int, d: int, scale: Optional[float] = None, causal: bool = False,
              dtype: Optional[torch.dtype] = None, device=None) -> torch.Tensor:
    """Inference entry point: the output only (cuda.go:125-139)."""
    return FlashAttnFwd(Q, K, V, BH, S, d, scale, causal, dtype, device)[0]


def FlashAttnBwd(Q, K, V, O, L, dO, BH: int, S: int, d: int, scale: Optional[float] = None,
                 causal: bool = False, dtype: Optional[torch.dtype] = None, device=None):
    """Returns ``(dQ, dK, dV)`` from the saved output and log-sum-exp, with the identities
    ``p = exp(s*scale - L)``, ``D = rowsum(dO * O)``, ``dV = p^T dO``, ``dS = p (dO V^T - D) scale``,
    ``dQ = dS K``, ``dK = dS^T Q`` (gonn_cuda.cu:333-340).  Deterministic: no atomics."""
    dev = _device(device)
    dt = _attn_dtype(dtype, dev, d)
    scale = (1.0 / math.sqrt(d)) if scale is None else float(scale)
    q, k, v, o, do = (_bshd(x, BH, S, d, dt, dev) for x in (Q, K, V, O, dO))
    lse = L._view(BH, S) if isinstance(L, DeviceBuffer) else torch.as_tensor(L).to(dev).reshape(BH, S)
    if _attn._kernel_ok(q, k, v):
        lse4 = lse.to(torch.float32).contiguous().view(1, BH, S)
        dq, dk, dv, _ = _attn.flash_bwd(q, k, v, o, do, lse4, bool(causal), scale)   # o is read through its strides
        return tuple(_flat(t, BH, S, d) for t in (dq, dk, dv))
    if _attn.general_ok(q, k, v):
        dq, dk, dv = _attn.general_bwd(q, k, v, o, do, lse.view(1, BH, S), bool(causal), scale)
        return tuple(_flat(t, BH, S, d) for t in (dq, dk, dv))
    ct = torch.float64 if dt == torch.float64 else torch.float32
    qf, kf, vf, of, dof = (_flat(t, BH, S, d).to(ct) for t in (q, k, v, o, do))
    s = torch.matmul(qf, kf.transpose(1, 2)) * scale
    if causal:
        s = s.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool, device=dev), diagonal=1), -1e30)
    p = torch.exp(s - lse.to(ct).unsqueeze(-1))
    delta = (dof * of).sum(-1, keepdim=True)
    dv = torch.matmul(p.transpose(1, 2), dof)
    ds = p * (torch.matmul(dof, vf.transpose(1, 2)) - delta) * scale
    return torch.matmul(ds, kf).to(dt), torch.matmul(ds.transpose(1, 2), qf).to(dt), dv.to(dt)


# -- device-resident benchmark loops ---------------------------------------------------------

def _time_ms(fn, iters: int, dev: torch.device) -> float:
    """Milliseconds per iteration: five warm-up calls, then ``iters`` calls between two CUDA
    events (``perf_counter`` on the host path)."""
    for _ in range(5):
        fn()
    if dev.type != "cuda":
        t0 = time.perf_counter()
        for _ in range(iters):
            fn()
        return (time.perf_counter() - t0) * 1e3 / iters
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def _native_loop(name: str, *args) -> float:
    """Runs one of the library's own benchmark loops (csrc/gemm_exact.cu): buffers, warm-up, the
    timed loop and the events all live on the native side, as in the reference's library."""
    ms = float(getattr(_l.lib(), name)(*args))
    if ms < 0:
        raise RuntimeError(f"{name}: device allocation or launch failed ({_l.lib().gb_last_error().decode()})")
    _l.kernel_count += 5 + int(args[-2].value)      # informational: launches made by the loop
    return ms


def BenchMatMulDev(m: int, k: int, n: int, iters: int, f32: bool = False, device=None) -> float:
    """Resident ``(m,k) @ (k,n)`` in float64 (float32 when ``f32``), ms per iteration."""
    dev = _device(device)
    if dev.type == "cuda":
        return _native_loop("gb_bench_matmul", _l.I(m), _l.I(k), _l.I(n), _l.I(iters), _l.I(2 if f32 else 3))
    dt = torch.float32 if f32 else torch.float64
    a, b = torch.randn(m, k, dtype=dt, device=dev), torch.randn(k, n, dtype=dt, device=dev)
    c = torch.empty(m, n, dtype=dt, device=dev)
    return _time_ms(lambda: _gemm(a, b, out=c), iters, dev)


def BenchMatMulF16Dev(m: int, k: int, n: int, iters: int, dtype: torch.dtype = torch.float16, device=None) -> float:
    dev = _device(device)
    if dev.type == "cuda":
        return _native_loop("gb_bench_matmul", _l.I(m), _l.I(k), _l.I(n), _l.I(iters),
                            _l.I(0 if dtype == torch.bfloat16 else 1))
    a, b = torch.randn(m, k, dtype=dtype, device=dev), torch.randn(k, n, dtype=dtype, device=dev)
    c = torch.empty(m, n, dtype=dtype, device=dev)
    return _time_ms(lambda: _gemm(a, b, out=c), iters, dev)


def BenchAddDev(n: int, iters: int, f32: bool = False, device=None) -> float:
    dev = _device(device)
    if dev.type == "cuda":
        return _native_loop("gb_bench_add", _l.L(n), _l.I(iters), _l.I(int(f32)))
    dt = torch.float32 if f32 else torch.float64
    a, b = torch.randn(n, dtype=dt, device=dev), torch.randn(n, dtype=dt, device=dev)
    return _time_ms(lambda: _ew.binary_forward("add", a, b), iters, dev)


def BenchFlashAttn(BH: int, S: int, d: int, iters: int, causal: bool = False,
                   dtype: Optional[torch.dtype] = None, device=None) -> float:
    """Forward attention on resident ``(BH, S, d)`` inputs, ms per iteration."""
    dev = _device(device)
    dt = _attn_dtype(dtype, dev, d)
    if dev.type == "cuda" and dt == torch.bfloat16 and d in (64, 128):
        return _native_loop("gb_bench_flash_attn", _l.I(BH), _l.I(S), _l.I(d), _l.I(iters), _l.I(int(causal)))
    q, k, v = (torch.randn(BH, S, d, dtype=dt, device=dev) for _ in range(3))
    q4, k4, v4 = (_bshd(t, BH, S, d, dt, dev) for t in (q, k, v))
    if _attn._kernel_ok(q4, k4, v4):
        # the loop runs the kernel alone on resident buffers, as the reference's in-library
        # benchmark does (gonn_cuda.cu:532-560): views and the output are prepared once
        o = torch.empty(BH, S, d, dtype=dt, device=dev).permute(1, 0, 2).unsqueeze(0)
        scale = 1.0 / math.sqrt(d)
        return _time_ms(lambda: _attn.flash_fwd(q4, k4, v4, bool(causal), scale, out=o), iters, dev)
    return _time_ms(lambda: FlashAttnFwd(q, k, v, BH, S, d, None, causal, dt, dev), iters, dev)


# the reference's names (its kernels are float64-only, hence the suffix); pass dtype=torch.float64
# for float64 arithmetic, leave it unset for the tensor-core path on 16-bit data
FlashAttnF64, FlashAttnF64Fwd, FlashAttnF64Bwd, BenchFlashAttnF64 = FlashAttn, FlashAttnFwd, FlashAttnBwd, BenchFlashAttn

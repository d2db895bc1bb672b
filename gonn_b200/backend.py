"""Compute-backend contract (backend/backend.go:18-117).

The reference selects a process-wide ``Backend`` (CPU / CUDA / OpenCL) with an atomic
``Use`` / ``Current`` and dispatches GEMM and, optionally, elementwise kinds to it.  This
framework has one accelerator path — the sm_100a kernels — and places work by the tensor's
device, so the contract is kept as an API: ``Current()`` describes what runs, ``Use`` swaps in
another object implementing ``Gemm`` (tests use a counting fake), and the kind enumerations
keep the reference's append-only numbering (they are a C ABI there).
"""
from __future__ import annotations

import enum
import threading
from typing import Optional

import torch

from .ops.gemm import gemm as _gemm
from .ops import elementwise as _ew


class Device(str, enum.Enum):
    CPU = "cpu"
    CUDA = "cuda"
    OPENCL = "opencl"


class UnaryKind(enum.IntEnum):
    NoneKind = -1
    ReLU = 0
    Sigmoid = 1
    Tanh = 2
    Exp = 3
    Log = 4
    GELU = 5
    SiLU = 6
    GELUExact = 7


class BinaryKind(enum.IntEnum):
    Add = 0
    Sub = 1
    Mul = 2
    Div = 3


_UNARY = {UnaryKind.ReLU: "relu", UnaryKind.Sigmoid: "sigmoid", UnaryKind.Tanh: "tanh", UnaryKind.Exp: "exp",
          UnaryKind.Log: "log", UnaryKind.GELU: "gelu", UnaryKind.SiLU: "silu", UnaryKind.GELUExact: "geluexact"}
_BINARY = {BinaryKind.Add: "add", BinaryKind.Sub: "sub", BinaryKind.Mul: "mul", BinaryKind.Div: "div"}


class Backend:
    """``Gemm(a, b, batch, m, k, n, transA, transB)`` on row-major, contiguous batches; op(A) is
    (m, k) and is stored (k, m) when ``transA``.  ``Unary`` / ``Binary`` may decline (return None)."""

    def Name(self) -> str:
        raise NotImplementedError

    def Gemm(self, a, b, batch, m, k, n, transA=False, transB=False):
        raise NotImplementedError

    def Synchronize(self) -> None:
        pass


class Elementwiser:
    """Optional capability (backend/backend.go:89-92): a backend that also evaluates the
    enum-dispatched elementwise kinds.  ``Unary`` / ``Binary`` return the result, or None to
    decline, in which case the caller evaluates the op on the host path."""

    def Unary(self, kind: "UnaryKind", x):
        return None

    def Binary(self, kind: "BinaryKind", a, b):
        return None


class NativeBackend(Backend, Elementwiser):
    def __init__(self, device: str):
        self.device = device

    def Name(self):
        return "sm_100a" if self.device == "cuda" else "cpu"

    def Gemm(self, a, b, batch, m, k, n, transA=False, transB=False):
        sa = (batch, k, m) if transA else (batch, m, k)
        sb = (batch, n, k) if transB else (batch, k, n)
        out = _gemm(a.reshape(sa), b.reshape(sb), trans_a=transA, trans_b=transB)
        return out.reshape(batch, m, n)

    def Unary(self, kind: UnaryKind, x):
        name = _UNARY.get(kind)
        return None if name is None else _ew.unary_forward(name, x)

    def Binary(self, kind: BinaryKind, a, b):
        return _ew.binary_forward(_BINARY[kind], a, b)

    def Synchronize(self):
        if self.device == "cuda":
            torch.cuda.synchronize()


_lock = threading.Lock()
_current: Optional[Backend] = None


def NewCPU() -> Backend:
    return NativeBackend("cpu")


def NewCUDA() -> Backend:
    if not torch.cuda.is_available():
        raise RuntimeError("backend.NewCUDA: no CUDA device")
    return NativeBackend("cuda")


def Use(b: Backend) -> Backend:
    """Installs ``b`` and returns the previous backend (atomic swap)."""
    global _current
    with _lock:
        prev = _current if _current is not None else NewCPU()
        _current = b
    return prev


def Current() -> Backend:
    global _current
    with _lock:
        if _current is None:
            _current = NewCPU()
        return _current

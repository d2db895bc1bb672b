"""ctypes binding of the native library (``_C/libgonn_b200.so``).

The library exposes a plain C ABI: raw device pointers, sizes and a CUDA stream
handle go in, an ``int`` status comes out (0 = success, negative = error with
text available from ``gb_last_error``).  PyTorch owns the storage and the
streams; the functions here only launch kernels on the current stream.

If a CUDA device is present and the library cannot be loaded, :func:`lib`
raises: GPU ops never fall back to another implementation silently.
"""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_double, c_float, c_int, c_longlong, c_void_p

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# GONN_B200_DEBUG=1 selects the bounds-checked build (python -m gonn_b200.build --debug): its window,
# embedding, reduction and normalisation kernels report an out-of-range index through the status word.
DEBUG_BUILD = os.environ.get("GONN_B200_DEBUG", "") not in ("", "0")
LIB_PATH = os.path.join(_HERE, "_C", "libgonn_b200_debug.so" if DEBUG_BUILD else "libgonn_b200.so")
# GONN_B200_LIB=<path> loads another build of the library (to compare two builds in one session)
LIB_PATH = os.environ.get("GONN_B200_LIB", LIB_PATH)

DT_BF16, DT_F16, DT_F32, DT_F64, DT_I8 = 0, 1, 2, 3, 4
_DT = {torch.bfloat16: DT_BF16, torch.float16: DT_F16, torch.float32: DT_F32,
       torch.float64: DT_F64, torch.int8: DT_I8}

_lib = None
_lock = threading.Lock()
launch_count = 0  # native entry points called through this binding
kernel_count = 0  # kernels those calls launched (read by bench.py)

# kernels launched per entry point when it is not exactly one
KERNELS_PER_CALL = {
    "gb_norm_bwd": 2, "gb_channel_sum": 2, "gb_ce_fwd": 2, "gb_ce_fused": 2, "gb_flash_bwd": 2, "gb_flash_bwd_ws": 2, "gb_embedding_bwd": 5,
    "gb_status_read": 0, "gb_comm_alloc": 0, "gb_comm_open": 0, "gb_comm_emulate": 0,
    "gb_comm_free": 0, "gb_reduce": 1, "gb_gemm_f32x3": 5, "gb_conv_wgrad": 2, "gb_set_words": 1, "gb_norm_bwd_res": 2,
}


class NativeError(RuntimeError):
    """A native entry point returned a non-zero status."""


class KernelStatusError(RuntimeError):
    """A kernel recorded an error (for example a wait that ran out of budget)."""


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DT[dt]
    except KeyError:
        raise TypeError(f"dtype {dt} is not supported by the native kernels") from None


def available() -> bool:
    """True when the shared object exists on disk (it may still need a GPU to run)."""
    return os.path.exists(LIB_PATH)


def lib() -> ctypes.CDLL:
    """Loads the library on first use (building is done by ``gonn_b200.build``)."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise NativeError(
                    f"{LIB_PATH} is missing: run `python -m gonn_b200.build` first")
            l = ctypes.CDLL(LIB_PATH)
            l.gb_last_error.restype = ctypes.c_char_p
            l.gb_gemm_f32x3_workspace.restype = c_longlong
            l.gb_gemm_f32x3_workspace.argtypes = [c_int, c_int, c_int, c_int]
            for name in ("gb_bench_matmul", "gb_bench_add", "gb_bench_flash_attn"):
                getattr(l, name).restype = c_double
            _lib = l
    return _lib


def use_native(t: torch.Tensor) -> bool:
    """CUDA tensors run on the native kernels; CPU tensors on the torch oracle path."""
    return t.is_cuda


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def current_stream_handle() -> int:
    """The current CUDA stream of the current device as an integer handle.  The private torch
    entry points are an order of magnitude cheaper than ``torch.cuda.current_stream()`` (which
    builds a Stream object: about 16 us per call, 5 ms per training step of the 12-layer LM);
    the public API is the fallback."""
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def stream_ptr() -> c_void_p:
    return c_void_p(current_stream_handle())


def ptr(t) -> c_void_p:
    if t is None:
        return c_void_p(0)
    return c_void_p(t.data_ptr())


def check(rc: int, what: str = "native call") -> None:
    if rc != 0:
        msg = lib().gb_last_error().decode(errors="replace")
        raise NativeError(f"{what} failed ({rc}): {msg}")


_fn_cache = {}
_call_hook = None


def set_call_hook(hook) -> None:
    """Installs ``hook(name, fn, args) -> status`` around every native call (``None`` removes
    it).  Used by ``gonn_b200.utils.trace``; the hook must call ``fn(*args)`` itself."""
    global _call_hook
    _call_hook = hook


def call(name: str, *args) -> None:
    """Calls ``name`` with ctypes-converted ``args`` and raises on a non-zero status."""
    global launch_count, kernel_count
    fn = _fn_cache.get(name)
    if fn is None:
        fn = _fn_cache[name] = getattr(lib(), name)
    rc = fn(*args) if _call_hook is None else _call_hook(name, fn, args)
    launch_count += 1
    kernel_count += KERNELS_PER_CALL.get(name, 1)
    if rc != 0:
        check(rc, name)


def read_status(clear: bool = True):
    """Returns the device status word ``(code, detail, block, count)`` (synchronises)."""
    buf = (c_int * 4)()
    check(lib().gb_status_read(buf, c_int(1 if clear else 0)), "gb_status_read")
    return tuple(buf)


def assert_status_ok() -> None:
    code, detail, block, count = read_status()
    if code != 0:
        raise KernelStatusError(
            f"kernel status code {code} (detail {detail}, block {block}, {count} reports)")


I = c_int
L = c_longlong
F = c_float
D = c_double
P = c_void_p

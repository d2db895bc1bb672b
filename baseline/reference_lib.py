"""The reference's own CUDA library, built unchanged and driven through its C ABI.

``backend/cuda/gonn_cuda.cu`` of the reference is a standalone file (CUDA runtime + cuBLAS,
no Go).  ``build()`` compiles it, unmodified, for sm_100 into ``baseline/_ref/libgonn_cuda.so``;
``load()`` opens that file with ``ctypes`` and declares the prototypes of
``backend/cuda/gonn_cuda.h:30-89``.  Nothing of this framework is imported here: the
functions below are the reference's stock code path (cuBLAS S/D/H GEMM, its elementwise and
flash-attention kernels, its in-library benchmark loops).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from ctypes import POINTER, c_double, c_int, c_long, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT_DIR, "libgonn_cuda.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")


def find_source() -> str | None:
    """Path of the reference's ``gonn_cuda.cu``: under ``$GONN_REFERENCE``, else under the default checkout location."""
    for root in (os.environ.get("GONN_REFERENCE"), "/root/reference"):
        if root:
            p = os.path.join(root, "backend", "cuda", "gonn_cuda.cu")
            if os.path.exists(p):
                return p
    return None


def build(force: bool = False) -> str | None:
    """Compiles the reference source (as is) into ``baseline/_ref/libgonn_cuda.so``.  Returns
    the path, or None when the source tree is not present (then an earlier build is kept)."""
    src = find_source()
    if src is None:
        return LIB if os.path.exists(LIB) else None
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(src):
        return LIB
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = [NVCC, "-O3", "-gencode", "arch=compute_100,code=sm_100", "-Xcompiler", "-fPIC", "-shared",
           src, "-o", LIB, "-lcublas"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed on the reference's gonn_cuda.cu:\n" + r.stdout + r.stderr)
    return LIB


_lib = None


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB):
        raise FileNotFoundError(LIB)
    l = ctypes.CDLL(LIB)
    dp = POINTER(c_double)
    l.gonn_gemm.argtypes = [dp, dp, dp, c_int, c_int, c_int, c_int, c_int, c_int]
    l.gonn_gemm.restype = c_int
    l.gonn_unary.argtypes = [c_int, dp, dp, c_long]
    l.gonn_unary.restype = c_int
    l.gonn_binary.argtypes = [c_int, dp, dp, dp, c_long]
    l.gonn_binary.restype = c_int
    l.gonn_sync.restype = None
    l.gonn_bench_matmul_dev.argtypes = [c_int, c_int, c_int, c_int, c_int]
    l.gonn_bench_matmul_dev.restype = c_double
    l.gonn_bench_matmul_f16_dev.argtypes = [c_int, c_int, c_int, c_int]
    l.gonn_bench_matmul_f16_dev.restype = c_double
    l.gonn_bench_add_dev.argtypes = [c_int, c_int, c_int]
    l.gonn_bench_add_dev.restype = c_double
    l.gonn_bench_flash_attn_f64.argtypes = [c_int, c_int, c_int, c_int, c_int]
    l.gonn_bench_flash_attn_f64.restype = c_double
    l.gonn_flash_attn_f64.argtypes = [dp, dp, dp, dp, c_int, c_int, c_int, c_double, c_int]
    l.gonn_flash_attn_f64.restype = None
    l.gonn_flash_attn_f64_fwd.argtypes = [dp, dp, dp, dp, dp, c_int, c_int, c_int, c_double, c_int]
    l.gonn_flash_attn_f64_fwd.restype = None
    l.gonn_flash_attn_f64_bwd.argtypes = [dp] * 9 + [c_int, c_int, c_int, c_double, c_int]
    l.gonn_flash_attn_f64_bwd.restype = None
    l.gonn_dev_alloc.argtypes = [c_long]
    l.gonn_dev_alloc.restype = c_void_p
    l.gonn_dev_free.argtypes = [c_void_p]
    l.gonn_dev_free.restype = None
    l.gonn_dev_upload.argtypes = [c_void_p, dp, c_long]
    l.gonn_dev_upload.restype = None
    l.gonn_dev_download.argtypes = [dp, c_void_p, c_long]
    l.gonn_dev_download.restype = None
    l.gonn_dev_sync.restype = None
    l.gonn_dev_matmul_f64.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int]
    l.gonn_dev_matmul_f64.restype = None
    l.gonn_dev_add_f64.argtypes = [c_void_p, c_void_p, c_void_p, c_int]
    l.gonn_dev_add_f64.restype = None
    l.gonn_dev_relu_f64.argtypes = [c_void_p, c_int]
    l.gonn_dev_relu_f64.restype = None
    _lib = l
    return l


def dptr(a):
    """``double*`` of a contiguous float64 numpy array."""
    return a.ctypes.data_as(POINTER(c_double))


if __name__ == "__main__":
    print(build(force=True))

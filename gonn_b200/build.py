"""Builds the native library ``gonn_b200/_C/libgonn_b200.so`` for sm_100a.

Every ``csrc/*.cu`` file is one translation unit compiled by ``nvcc`` with
``-gencode arch=compute_100a,code=sm_100a`` and linked into one shared object
with a C ABI (loaded through ``ctypes`` by :mod:`gonn_b200.lib`).  No GPU is
needed to build.  Run ``python -m gonn_b200.build`` (add ``-v`` for
``-Xptxas -v`` resource usage, ``-f`` to force a full rebuild).  The reference compiles its one CUDA
source with a single ``nvcc -O3 -arch=sm_86 ... -lcublas`` line
(benchmark/docker/build_and_run.sh:14); here objects are cached by a digest of source, headers and
flags, so a change recompiles one unit.

``python -m gonn_b200.build --debug`` builds a second library,
``libgonn_b200_debug.so``, with ``-DGB_BOUNDS_CHECK``: the window, embedding, reduction and
normalisation kernels then check every data-dependent or computed index against the extent of
its buffer and report a violation through the status word instead of making the access
(``csrc/bounds.cuh``).  ``GONN_B200_DEBUG=1`` makes :mod:`gonn_b200.lib` load that library.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(HERE, "_C")
OBJ_DIR = os.path.join(OUT_DIR, "obj")
LIB = os.path.join(OUT_DIR, "libgonn_b200.so")
DEBUG_LIB = os.path.join(OUT_DIR, "libgonn_b200_debug.so")
DEBUG_FLAGS = ["-DGB_BOUNDS_CHECK"]

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "--use_fast_math", "-Xcompiler", "-fPIC",
          "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr", "-I", CSRC]


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _digest(path: str, extra=()) -> str:
    h = hashlib.sha256()
    for name in sorted(os.listdir(CSRC)):
        if name.endswith((".cuh", ".h")):
            with open(os.path.join(CSRC, name), "rb") as f:
                h.update(f.read())
    with open(path, "rb") as f:
        h.update(f.read())
    h.update(" ".join(ARCH + COMMON + list(extra)).encode())
    return h.hexdigest()


def _has_checks(name: str) -> bool:
    """Whether the translation unit changes under -DGB_BOUNDS_CHECK (it includes bounds.cuh or tests the macro)."""
    with open(os.path.join(CSRC, name)) as f:
        text = f.read()
    return "bounds.cuh" in text or "GB_BOUNDS_CHECK" in text


def _compile(name: str, verbose: bool, force: bool, debug: bool = False):
    src = os.path.join(CSRC, name)
    if debug and not _has_checks(name):
        debug = False              # identical object either way: the debug library links the regular one
    extra = DEBUG_FLAGS if debug else []
    obj = os.path.join(OBJ_DIR, name[:-3] + (".dbg.o" if debug else ".o"))
    stamp = obj + ".sha"
    dig = _digest(src, extra)
    if not force and os.path.exists(obj) and os.path.exists(stamp):
        with open(stamp) as f:
            if f.read().strip() == dig:
                return name, False, ""
    cmd = [NVCC] + ARCH + COMMON + extra + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {name}:\n{r.stdout}\n{r.stderr}")
    with open(stamp, "w") as f:
        f.write(dig)
    return name, True, r.stderr


def build(verbose: bool = False, force: bool = False, debug: bool = False) -> str:
    """Compiles what changed and links the shared library (the bounds-checked one when ``debug``);
    returns its path."""
    os.makedirs(OBJ_DIR, exist_ok=True)
    srcs = _sources()
    rebuilt = False
    lib = DEBUG_LIB if debug else LIB
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        for name, did, log in ex.map(lambda n: _compile(n, verbose, force, debug), srcs):
            rebuilt |= did
            if verbose and log:
                print(f"--- {name}\n{log}")
    objs = [os.path.join(OBJ_DIR, n[:-3] + (".dbg.o" if debug and _has_checks(n) else ".o")) for n in srcs]
    # an object may have been rebuilt by the other flavour's pass (the two libraries share most objects)
    if rebuilt or not os.path.exists(lib) or any(os.path.getmtime(o) > os.path.getmtime(lib) for o in objs):
        cmd = [NVCC] + ARCH + ["-shared", "-o", lib] + objs + ["-lcudart", "-lpthread"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return lib


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force="-f" in sys.argv, debug="--debug" in sys.argv)
    print(path)

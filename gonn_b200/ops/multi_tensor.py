"""Multi-tensor launches of the fused optimizer kernels (csrc/optim.cu).

The update rules are the reference's per-element loops (optim/sgd.go:47-69, adam.go:61-77,
adamw.go:64-84, lion.go:61-76, lamb.go:73-108) and its global-norm clipping (optim/clip.go:23-65);
one launch updates up to 48 tensors in chunks of 4096 elements instead of one host loop per
parameter."""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import torch

from .. import lib as _l

SGD, ADAM, LION, LAMB1, LAMB2, SQNORM, SCALE = range(7)
_MAXT = 48
_CHUNK = 4096


def _ptr_array(ts: Optional[Sequence[Optional[torch.Tensor]]], n: int):
    arr = (ctypes.c_void_p * n)()
    if ts is not None:
        for i, t in enumerate(ts):
            arr[i] = t.data_ptr() if t is not None else None
    return arr


def launch(algo: int, params: List[torch.Tensor], grads: List[torch.Tensor], masters, state0, state1,
           hyper: Sequence[float], flags: int = 0, aux: Optional[torch.Tensor] = None, aux_stride: int = 0):
    """Runs ``algo`` over the tensors (all of one dtype), ``_MAXT`` per launch.

    ``aux_stride``: floats of ``aux`` consumed per tensor (LAMB) — the aux pointer advances
    with each launch; for SQNORM aux advances by the number of chunks.
    """
    if not params:
        return
    dt = _l.dtype_code(params[0].dtype)
    hy = (ctypes.c_float * 9)(*[float(h) for h in hyper])
    aux_off = 0
    for i0 in range(0, len(params), _MAXT):
        ps = params[i0:i0 + _MAXT]
        n = len(ps)
        numel = (ctypes.c_longlong * n)(*[p.numel() for p in ps])
        sl = slice(i0, i0 + _MAXT)
        auxp = None
        if aux is not None:
            auxp = ctypes.c_void_p(aux.data_ptr() + 4 * aux_off)
        _l.call("gb_multi_tensor", _l.I(algo), _l.I(dt), _l.I(n), _ptr_array(ps, n),
                _ptr_array(grads[sl] if grads is not None else None, n),
                _ptr_array(masters[sl] if masters is not None else None, n),
                _ptr_array(state0[sl] if state0 is not None else None, n),
                _ptr_array(state1[sl] if state1 is not None else None, n),
                numel, hy, _l.I(flags), auxp, _l.stream_ptr())
        if algo == SQNORM:
            aux_off += sum((p.numel() + _CHUNK - 1) // _CHUNK for p in ps)
        else:
            aux_off += aux_stride * n


def chunks_of(ts: Sequence[torch.Tensor]) -> int:
    return sum((t.numel() + _CHUNK - 1) // _CHUNK for t in ts)


def by_dtype(params: Sequence[torch.Tensor]):
    groups = {}
    for p in params:
        groups.setdefault((p.dtype, p.device), []).append(p)
    return groups.values()


def native(p: torch.Tensor) -> bool:
    return p.is_cuda and p.dtype in (torch.bfloat16, torch.float16, torch.float32, torch.float64)

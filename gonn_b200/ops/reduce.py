"""Axis reductions (sum / mean / max / min / argmax / argmin) over one axis.

CUDA tensors use ``csrc/reduce.cu`` (the tensor is viewed as (outer, R, inner));
CPU tensors use torch.  Semantics follow tensor/ops_reduce.go:6-271: one axis at
a time, optional keepdim, first extremum wins for arg reductions.
"""
from __future__ import annotations

import torch

from .. import lib as _l

_OPS = {"sum": 0, "mean": 1, "max": 2, "min": 3, "argmax": 4, "argmin": 5}
_scratch = {}


def _get_scratch(device, nbytes: int) -> torch.Tensor:
    key = (device.type, device.index)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _scratch[key] = buf
    return buf


def reduce_axis(x: torch.Tensor, axis: int, op: str = "sum", keepdim: bool = False,
                out_dtype=None, out: torch.Tensor = None, accumulate: bool = False) -> torch.Tensor:
    """Reduces ``x`` over ``axis`` (no autograd; see tensor API for the differentiable forms)."""
    axis = axis % x.dim()
    if not (x.is_cuda and x.dtype in (torch.bfloat16, torch.float16, torch.float32, torch.float64)):
        if x.is_cuda:
            raise TypeError(f"reduce: no CUDA kernel for dtype {x.dtype}")
        if op in ("argmax", "argmin"):
            r = getattr(torch, op)(x, dim=axis, keepdim=keepdim)
        elif op in ("max", "min"):
            r = getattr(torch, op)(x, dim=axis, keepdim=keepdim).values
        else:
            xx = x if x.dtype in (torch.float32, torch.float64) else x.float()
            r = getattr(torch, op)(xx, dim=axis, keepdim=keepdim)
            r = r.to(out_dtype or x.dtype)
        if out is not None:
            if accumulate:
                out.add_(r.reshape(out.shape))
            else:
                out.copy_(r.reshape(out.shape))
            return out
        return r
    xc = x.contiguous()
    outer = 1
    for s in xc.shape[:axis]:
        outer *= s
    R = xc.shape[axis]
    inner = 1
    for s in xc.shape[axis + 1:]:
        inner *= s
    oshape = list(xc.shape)
    if keepdim:
        oshape[axis] = 1
    else:
        del oshape[axis]
    arg = op in ("argmax", "argmin")
    odt = torch.int64 if arg else (out.dtype if out is not None else (out_dtype or x.dtype))
    if out is None:
        out = torch.empty(oshape, dtype=odt, device=x.device)
        accumulate = False
    esz = 8 if x.dtype == torch.float64 else 4
    need = 0
    if inner > 1 and not arg:
        need = 148 * 8 * max(inner, 32) * esz + outer * inner * esz * (2 if accumulate else 1)
        need = min(need, 256 << 20)
    elif accumulate:
        need = outer * inner * esz
    scratch = _get_scratch(x.device, need) if need else None
    _l.call("gb_reduce", _l.I(_OPS[op]), _l.I(_l.dtype_code(x.dtype)),
            _l.I(_l.dtype_code(x.dtype) if arg else _l.dtype_code(odt)), _l.ptr(xc), _l.ptr(out), _l.ptr(scratch),
            _l.L(scratch.numel() if scratch is not None else 0), _l.L(outer), _l.L(R), _l.L(inner),
            _l.I(int(accumulate)), _l.stream_ptr())
    return out


def column_sum(x2d: torch.Tensor, out_dtype=None, out=None, accumulate=False) -> torch.Tensor:
    """Sum over rows of a (rows, cols) matrix: the bias-gradient reduction."""
    return reduce_axis(x2d, 0, "sum", out_dtype=out_dtype, out=out, accumulate=accumulate)

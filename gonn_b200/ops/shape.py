"""Materialised transpose and prefix sum (kernels in ``csrc/shape.cu``).

``transpose_last2(x)`` returns a contiguous tensor with the last two dimensions swapped
(tiled through shared memory); ``cumsum(x, axis)`` is an inclusive prefix sum with a
reverse-scan backward.  CPU tensors and unsupported dtypes use the torch expression.
"""
from __future__ import annotations

import torch

from .. import lib as _l

_SCAN_DTYPES = (torch.float32, torch.float64, torch.float16, torch.bfloat16)


def _transpose_kernel(x: torch.Tensor) -> torch.Tensor:
    xc = x.contiguous()
    R, C = xc.shape[-2], xc.shape[-1]
    batch = xc.numel() // (R * C) if R * C else 0
    out = torch.empty(xc.shape[:-2] + (C, R), dtype=x.dtype, device=x.device)
    if batch == 0:
        return out
    for lo in range(0, batch, 65535):   # gridDim.z limit
        n = min(65535, batch - lo)
        src = xc.reshape(batch, R, C)[lo:lo + n]
        dst = out.reshape(batch, C, R)[lo:lo + n]
        _l.call("gb_transpose2d", _l.I(x.element_size()), _l.ptr(src), _l.ptr(dst), _l.I(R), _l.I(C), _l.I(n),
                _l.stream_ptr())
    return out


class _Transpose(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return _transpose_kernel(x)

    @staticmethod
    def backward(ctx, g):
        return _transpose_kernel(g)


def transpose_last2(x: torch.Tensor) -> torch.Tensor:
    """Contiguous copy of ``x`` with its last two dimensions swapped."""
    if x.dim() < 2:
        raise ValueError("transpose_last2: needs at least two dimensions")
    if x.is_cuda and x.element_size() in (2, 4, 8) and not x.is_complex():
        return _Transpose.apply(x)
    return x.transpose(-1, -2).contiguous()


def _scan_kernel(x2: torch.Tensor, reverse: bool) -> torch.Tensor:
    y = torch.empty_like(x2)
    _l.call("gb_cumsum", _l.I(_l.dtype_code(x2.dtype)), _l.ptr(x2), _l.ptr(y), _l.L(x2.shape[0]), _l.L(x2.shape[1]),
            _l.I(int(reverse)), _l.stream_ptr())
    return y


class _Cumsum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2):
        return _scan_kernel(x2, False)

    @staticmethod
    def backward(ctx, g):
        # adjoint of an inclusive scan: the scan from the other end
        return _scan_kernel(g.contiguous(), True)


def cumsum(x: torch.Tensor, axis: int = -1) -> torch.Tensor:
    """Inclusive prefix sum along ``axis`` (tensor/ops_extra.go Cumsum of the reference)."""
    if not (x.is_cuda and x.dtype in _SCAN_DTYPES) or x.numel() == 0:
        return torch.cumsum(x, dim=axis)
    axis = axis % x.dim()
    last = x.dim() - 1
    xm = x if axis == last else x.movedim(axis, last)
    shape = xm.shape
    y = _Cumsum.apply(xm.contiguous().reshape(-1, shape[-1])).reshape(shape)
    return y if axis == last else y.movedim(last, axis)

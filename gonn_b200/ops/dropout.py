"""Dropout with a counter-based generator: the mask is a pure function of
(seed, offset, element index), so backward regenerates it instead of storing it.
CUDA: ``csrc/dropout.cu`` (Philox-4x32-10).  CPU: torch's generator.

Semantics of the reference's layer (nn/dropout.go:21-37: keep with probability 1 - p, scale the kept
values by 1 / (1 - p), identity in evaluation mode); the reference draws its mask on the host and
stores it, here nothing is stored."""
from __future__ import annotations

import torch

from .. import lib as _l

_counter = [0]


class _Dropout(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, p, seed, offset):
        xc = x.contiguous()
        y = torch.empty_like(xc)
        _l.call("gb_dropout", _l.I(_l.dtype_code(x.dtype)), _l.ptr(xc), _l.ptr(y), _l.L(xc.numel()),
                _l.F(p), _l.L(seed), _l.L(offset), _l.stream_ptr())
        ctx.meta = (p, seed, offset)
        return y

    @staticmethod
    def backward(ctx, dy):
        p, seed, offset = ctx.meta
        dyc = dy.contiguous()
        dx = torch.empty_like(dyc)
        _l.call("gb_dropout", _l.I(_l.dtype_code(dy.dtype)), _l.ptr(dyc), _l.ptr(dx), _l.L(dyc.numel()),
                _l.F(p), _l.L(seed), _l.L(offset), _l.stream_ptr())
        return dx, None, None, None


def dropout(x: torch.Tensor, p: float) -> torch.Tensor:
    if x.is_cuda and x.dtype in (torch.bfloat16, torch.float16, torch.float32):
        seed = int(torch.initial_seed() & 0x7FFFFFFFFFFFFFFF)
        _counter[0] += 1
        return _Dropout.apply(x, float(p), seed, _counter[0])
    mask = (torch.rand_like(x, dtype=torch.float32) >= p).to(x.dtype) / (1 - p)
    return x * mask

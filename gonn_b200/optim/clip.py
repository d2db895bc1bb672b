"""Gradient clipping and parameter <-> vector utilities (optim/clip.go:23-82,
optim/vecutil.go:22-81).  On CUDA the norm and the scaling run as multi-tensor kernels."""
from __future__ import annotations

import math
from typing import Sequence

import torch

from ..ops import multi_tensor as mt


def TotalGradNorm(params: Sequence[torch.Tensor], norm_type: float = 2.0) -> float:
    ps = [p for p in params if p.grad is not None]
    if not ps:
        return 0.0
    if norm_type == 2.0 and all(mt.native(p.grad) for p in ps):
        total = torch.zeros(1, dtype=torch.float32, device=ps[0].device)
        from .. import lib as _l
        for grp in mt.by_dtype([p.grad for p in ps]):
            part = torch.empty(mt.chunks_of(grp), dtype=torch.float32, device=grp[0].device)
            mt.launch(mt.SQNORM, grp, grp, None, None, None, [0, 0, 0, 0, 0, 1, 1, 0, 1.0], 0, part)
            _l.call("gb_sum_partials", _l.ptr(part), _l.I(part.numel()), _l.ptr(total), _l.I(1), _l.stream_ptr())
        return math.sqrt(float(total.item()))
    if norm_type == float("inf"):
        return max(float(p.grad.abs().max()) for p in ps)
    return float(sum(float(p.grad.double().abs().pow(norm_type).sum()) for p in ps) ** (1.0 / norm_type))


def ClipGradsWithNorm(params: Sequence[torch.Tensor], max_norm: float, norm: float) -> None:
    """Scales all gradients by max_norm / (norm + 1e-6) when that factor is below 1."""
    scale = max_norm / (norm + 1e-6)
    if scale >= 1.0:
        return
    gs = [p.grad for p in params if p.grad is not None]
    for grp in mt.by_dtype(gs):
        if mt.native(grp[0]):
            mt.launch(mt.SCALE, grp, grp, None, None, None, [0, 0, 0, 0, 0, 1, 1, 0, scale], 0)
        else:
            for g in grp:
                g.mul_(scale)


def ClipGradNorm(params: Sequence[torch.Tensor], max_norm: float, norm_type: float = 2.0) -> float:
    """Clips in place; returns the norm BEFORE clipping (for logging)."""
    params = list(params)
    norm = TotalGradNorm(params, norm_type)
    ClipGradsWithNorm(params, max_norm, norm)
    return norm


def ClipGradValue(params: Sequence[torch.Tensor], clip: float) -> None:
    for p in params:
        if p.grad is not None:
            p.grad.clamp_(-clip, clip)


def ParametersToVector(params: Sequence[torch.Tensor]) -> torch.Tensor:
    return torch.cat([p.detach().reshape(-1) for p in params])


def VectorToParameters(vec: torch.Tensor, params: Sequence[torch.Tensor]) -> None:
    n = sum(p.numel() for p in params)
    if vec.numel() != n:
        raise ValueError(f"VectorToParameters: vector has {vec.numel()} elements, parameters need {n}")
    off = 0
    with torch.no_grad():
        for p in params:
            k = p.numel()
            p.copy_(vec[off:off + k].reshape(p.shape).to(p.dtype))
            off += k


def GradsToVector(params: Sequence[torch.Tensor]) -> torch.Tensor:
    """Missing gradients contribute zeros."""
    return torch.cat([(p.grad if p.grad is not None else torch.zeros_like(p)).reshape(-1) for p in params])

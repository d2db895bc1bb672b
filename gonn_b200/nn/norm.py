"""Normalisation layers over the trailing dimension(s): LayerNorm, RMSNorm
(nn/norm.go:15-148).  Defaults: LayerNorm eps 1e-5, RMSNorm eps 1e-6 (weight only)."""
from __future__ import annotations

import torch

from ..ops.norm import layer_norm, rms_norm
from .module import Module


class LayerNorm(Module):
    def __init__(self, normalized_shape, eps: float = 1e-5, affine: bool = True, *, dtype=torch.float32,
                 device=None):
        super().__init__()
        if isinstance(normalized_shape, int):
            normalized_shape = (normalized_shape,)
        self.normalized_shape = tuple(normalized_shape)
        self.eps = eps
        n = 1
        for s in self.normalized_shape:
            n *= s
        self._n = n
        if affine:
            self.weight = torch.nn.Parameter(torch.ones(self.normalized_shape, dtype=dtype, device=device))
            self.bias = torch.nn.Parameter(torch.zeros(self.normalized_shape, dtype=dtype, device=device))
        else:
            self.weight = self.bias = None

    def forward(self, x):
        shp = x.shape
        nd = len(self.normalized_shape)
        if tuple(shp[-nd:]) != self.normalized_shape:
            raise ValueError(f"nn.LayerNorm: trailing dims {tuple(shp[-nd:])} != {self.normalized_shape}")
        x2 = x.reshape(-1, self._n)
        w = self.weight.reshape(-1) if self.weight is not None else None
        b = self.bias.reshape(-1) if self.bias is not None else None
        return layer_norm(x2, w, b, self.eps).reshape(shp)


class RMSNorm(Module):
    def __init__(self, dim: int, eps: float = 1e-6, *, dtype=torch.float32, device=None):
        super().__init__()
        self.dim, self.eps = dim, eps
        self.weight = torch.nn.Parameter(torch.ones(dim, dtype=dtype, device=device))

    def forward(self, x):
        shp = x.shape
        return rms_norm(x.reshape(-1, self.dim), self.weight, self.eps).reshape(shp)

"""Normalisation layers over the trailing dimension(s): LayerNorm, RMSNorm
(nn/norm.go:15-148).  Defaults: LayerNorm eps 1e-5, RMSNorm eps 1e-6 (weight only)."""
from __future__ import annotations

import torch

from ..ops.norm import fork_fuses, layer_norm, norm_fork, rms_norm
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
        return layer_norm(x2, self._flat(self.weight), self._flat(self.bias), self.eps).reshape(shp)

    @staticmethod
    def _flat(p):
        # a 1-D parameter is passed as itself: the kernels' gradient sinks are looked up on the
        # parameter object, which a reshaped alias would hide
        return None if p is None else (p if p.dim() == 1 else p.reshape(-1))

    def fork(self, x, res_bias=None):
        """``(self(x), x)`` for a block ``x + f(self(x))``: the backward adds the gradient that
        bypasses the norm inside the norm's own kernel and also yields the gradient of
        ``res_bias`` (see ``ops.norm.norm_fork``).  Returns None when that path does not apply."""
        if len(self.normalized_shape) != 1 or x.shape[-1] != self._n or not fork_fuses(x):
            return None
        y, xp = norm_fork(x.reshape(-1, self._n), self._flat(self.weight), self._flat(self.bias), self.eps, False,
                          res_bias)
        return y.reshape(x.shape), xp.reshape(x.shape)


class RMSNorm(Module):
    def __init__(self, dim: int, eps: float = 1e-6, *, dtype=torch.float32, device=None):
        super().__init__()
        self.dim, self.eps = dim, eps
        self.weight = torch.nn.Parameter(torch.ones(dim, dtype=dtype, device=device))

    def forward(self, x):
        shp = x.shape
        return rms_norm(x.reshape(-1, self.dim), self.weight, self.eps).reshape(shp)

    def fork(self, x, res_bias=None):
        """``(self(x), x)`` with the fused backward of ``LayerNorm.fork``."""
        if x.shape[-1] != self.dim or not fork_fuses(x):
            return None
        y, xp = norm_fork(x.reshape(-1, self.dim), self.weight, None, self.eps, True, res_bias)
        return y.reshape(x.shape), xp.reshape(x.shape)

"""BatchNorm1d/2d/3d, InstanceNorm1d/2d/3d, GroupNorm, LocalResponseNorm
(nn/batchnorm.go:13-123, nn/norm.go:150-266, nn/norm3d.go, nn/lrn.go).

Buffers ``running_mean`` / ``running_var`` (no ``num_batches_tracked``); eps 1e-5,
momentum 0.1; the running variance uses n/(n-1).  ``fused_relu`` applies ReLU inside
the normalise kernel."""
from __future__ import annotations

import torch

from ..ops.batchnorm import batch_norm_eval, batch_norm_train
from .module import Module


class _BatchNormNd(Module):
    ranks = (4,)

    def __init__(self, num_features: int, eps: float = 1e-5, momentum: float = 0.1, affine: bool = True,
                 fused_relu: bool = False, *, dtype=torch.float32, device=None):
        super().__init__()
        self.num_features, self.eps, self.momentum, self.fused_relu = num_features, eps, momentum, fused_relu
        if affine:
            self.weight = torch.nn.Parameter(torch.ones(num_features, dtype=dtype, device=device))
            self.bias = torch.nn.Parameter(torch.zeros(num_features, dtype=dtype, device=device))
        else:
            self.weight = self.bias = None
        sdt = torch.float64 if dtype == torch.float64 else torch.float32
        self.register_buffer("running_mean", torch.zeros(num_features, dtype=sdt, device=device))
        self.register_buffer("running_var", torch.ones(num_features, dtype=sdt, device=device))

    def _sync(self):
        return None, None

    def forward(self, x):
        if x.dim() not in self.ranks or x.shape[1] != self.num_features:
            raise ValueError(f"{type(self).__name__}: expected (N, {self.num_features}, ...) of rank {self.ranks}")
        if self.training:
            sync, group = self._sync()
            return batch_norm_train(x, self.weight, self.bias, self.running_mean, self.running_var, self.eps,
                                    self.momentum, self.fused_relu, sync, group)
        return batch_norm_eval(x, self.weight, self.bias, self.running_mean, self.running_var, self.eps,
                               self.fused_relu)


class BatchNorm1d(_BatchNormNd):
    ranks = (2, 3)


class BatchNorm2d(_BatchNormNd):
    ranks = (4,)


class BatchNorm3d(_BatchNormNd):
    ranks = (5,)


class GroupNorm(Module):
    """Normalises over (channels/groups, spatial) per sample; affine per channel."""

    def __init__(self, num_groups: int, num_channels: int, eps: float = 1e-5, affine: bool = True, *,
                 dtype=torch.float32, device=None):
        super().__init__()
        if num_channels % num_groups:
            raise ValueError("GroupNorm: channels must be divisible by groups")
        self.num_groups, self.num_channels, self.eps = num_groups, num_channels, eps
        if affine:
            self.weight = torch.nn.Parameter(torch.ones(num_channels, dtype=dtype, device=device))
            self.bias = torch.nn.Parameter(torch.zeros(num_channels, dtype=dtype, device=device))
        else:
            self.weight = self.bias = None

    def forward(self, x):
        from ..ops.norm import layer_norm
        N, C = x.shape[:2]
        g = self.num_groups
        y = layer_norm(x.reshape(N * g, -1), None, None, self.eps).reshape(x.shape)
        if self.weight is not None:
            shape = [1, C] + [1] * (x.dim() - 2)
            y = y * self.weight.reshape(shape) + self.bias.reshape(shape)
        return y


class _InstanceNormNd(Module):
    rank = 4

    def __init__(self, num_features: int, eps: float = 1e-5, affine: bool = False, *, dtype=torch.float32,
                 device=None):
        super().__init__()
        self.num_features, self.eps = num_features, eps
        if affine:
            self.weight = torch.nn.Parameter(torch.ones(num_features, dtype=dtype, device=device))
            self.bias = torch.nn.Parameter(torch.zeros(num_features, dtype=dtype, device=device))
        else:
            self.weight = self.bias = None

    def forward(self, x):
        from ..ops.norm import layer_norm
        if x.dim() != self.rank:
            raise ValueError(f"{type(self).__name__}: expected rank {self.rank}")
        N, C = x.shape[:2]
        y = layer_norm(x.reshape(N * C, -1), None, None, self.eps).reshape(x.shape)
        if self.weight is not None:
            shape = [1, C] + [1] * (x.dim() - 2)
            y = y * self.weight.reshape(shape) + self.bias.reshape(shape)
        return y


class InstanceNorm1d(_InstanceNormNd):
    rank = 3


class InstanceNorm2d(_InstanceNormNd):
    rank = 4


class InstanceNorm3d(_InstanceNormNd):
    rank = 5


class LocalResponseNorm(Module):
    """x / (k + alpha/n * sum_{window} x^2)^beta over channels, window [c - n/2, c + (n-1)/2]
    clamped, divisor always n (nn/lrn.go:52-92)."""

    def __init__(self, size: int, alpha: float = 1e-4, beta: float = 0.75, k: float = 1.0):
        super().__init__()
        self.size, self.alpha, self.beta, self.k = size, alpha, beta, k

    def forward(self, x):
        C = x.shape[1]
        sq = x * x
        lo, hi = self.size // 2, (self.size - 1) // 2
        pad = torch.nn.functional.pad(sq.transpose(1, -1), (lo, hi)).transpose(1, -1)
        acc = sum(pad.narrow(1, i, C) for i in range(self.size))
        return x / (self.k + self.alpha / self.size * acc) ** self.beta

"""Lazy modules: the first forward infers the input feature / channel count, builds the real
layer (random numbers are drawn at that moment), registers it as child ``inner`` and keeps
train / eval in sync (nn/lazy.go:35-357)."""
from __future__ import annotations

import torch

from . import batchnorm as _bn
from . import conv as _conv
from .linear import Linear
from .module import Module


class _Lazy(Module):
    def __init__(self, build, dim_of):
        super().__init__()
        self._build, self._dim_of = build, dim_of
        self.inner = None

    def IsInitialized(self) -> bool:
        return self.inner is not None

    def InnerModule(self):
        return self.inner

    Inner = InnerModule

    def forward(self, x):
        if self.inner is None:
            m = self._build(self._dim_of(x)).to(device=x.device)
            if x.dtype.is_floating_point:
                m = m.to(dtype=x.dtype)
            m.train(self.training)
            self.inner = m          # registered as child "inner"
        return self.inner(x)


def IsLazy(m) -> bool:
    return isinstance(m, _Lazy) and m.inner is None


def _chan(x):
    if x.dim() < 2:
        raise ValueError("lazy module: input needs a channel dimension")
    return x.shape[1]


def LazyLinear(out_features: int, bias: bool = True):
    return _Lazy(lambda n: Linear(n, out_features, bias), lambda x: x.shape[-1])


def _lazy_conv(cls):
    def make(out_channels, kernel_size, **kw):
        return _Lazy(lambda c: cls(c, out_channels, kernel_size, **kw), _chan)
    make.__name__ = "Lazy" + cls.__name__
    return make


LazyConv1d, LazyConv2d, LazyConv3d = (_lazy_conv(c) for c in (_conv.Conv1d, _conv.Conv2d, _conv.Conv3d))
LazyConvTranspose1d, LazyConvTranspose2d, LazyConvTranspose3d = (
    _lazy_conv(c) for c in (_conv.ConvTranspose1d, _conv.ConvTranspose2d, _conv.ConvTranspose3d))


def _lazy_norm(cls):
    def make(**kw):
        return _Lazy(lambda c: cls(c, **kw), _chan)
    make.__name__ = "Lazy" + cls.__name__
    return make


LazyBatchNorm1d, LazyBatchNorm2d, LazyBatchNorm3d = (
    _lazy_norm(c) for c in (_bn.BatchNorm1d, _bn.BatchNorm2d, _bn.BatchNorm3d))
LazyInstanceNorm1d, LazyInstanceNorm2d, LazyInstanceNorm3d = (
    _lazy_norm(c) for c in (_bn.InstanceNorm1d, _bn.InstanceNorm2d, _bn.InstanceNorm3d))

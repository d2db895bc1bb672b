"""Dropout family (nn/dropout.go:12-37, nn/dropout_channel.go:24-205)."""
from __future__ import annotations

import math

import torch

from .module import Module


class Dropout(Module):
    """Inverted dropout: survivors scaled by 1/(1-p) in training; identity in eval."""

    def __init__(self, p: float = 0.5):
        super().__init__()
        if not 0.0 <= p < 1.0:
            raise ValueError("nn.Dropout: p must be in [0, 1)")
        self.p = p

    def forward(self, x):
        if not self.training or self.p == 0.0:
            return x
        from ..ops.dropout import dropout
        return dropout(x, self.p)


class _ChannelDropout(Module):
    rank = None

    def __init__(self, p: float = 0.5):
        super().__init__()
        self.p = p

    def forward(self, x):
        if x.dim() != self.rank + 2:
            raise ValueError(f"{type(self).__name__}: expected a {self.rank + 2}-D input (N, C, ...)")
        if not self.training or self.p == 0.0:
            return x
        shape = list(x.shape[:2]) + [1] * self.rank
        mask = (torch.rand(shape, device=x.device) >= self.p).to(x.dtype) / (1 - self.p)
        return x * mask


class Dropout1d(_ChannelDropout):
    rank = 1


class Dropout2d(_ChannelDropout):
    rank = 2


class Dropout3d(_ChannelDropout):
    rank = 3


_ALPHA_P = -1.7580993408473766


class AlphaDropout(Module):
    """Keeps self-normalising statistics: a * (x*mask + alpha'(1-mask)) + b."""

    feature = False

    def __init__(self, p: float = 0.5):
        super().__init__()
        self.p = p

    def forward(self, x):
        if not self.training or self.p == 0.0:
            return x
        q = 1 - self.p
        a = (q + _ALPHA_P ** 2 * q * (1 - q)) ** -0.5
        b = -a * _ALPHA_P * (1 - q)
        shape = list(x.shape[:2]) + [1] * (x.dim() - 2) if self.feature else list(x.shape)
        mask = (torch.rand(shape, device=x.device) >= self.p).to(x.dtype)
        return a * (x * mask + _ALPHA_P * (1 - mask)) + b


class FeatureAlphaDropout(AlphaDropout):
    feature = True

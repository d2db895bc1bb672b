"""Evaluation-time fusion of a layer with the BatchNorm that follows it (nn/fuse.go:29-72):
w' = w * gamma / sqrt(var + eps), b' = (b - mean) * gamma / sqrt(var + eps) + beta."""
from __future__ import annotations

import torch

from .batchnorm import BatchNorm1d, BatchNorm2d
from .conv import Conv2d
from .linear import Linear


def _scale_shift(bn):
    inv = torch.rsqrt(bn.running_var + bn.eps)
    gamma = bn.weight.detach().to(inv.dtype) if bn.weight is not None else torch.ones_like(inv)
    beta = bn.bias.detach().to(inv.dtype) if bn.bias is not None else torch.zeros_like(inv)
    return gamma * inv, beta - bn.running_mean * gamma * inv


@torch.no_grad()
def FuseConvBNEval(conv: Conv2d, bn: BatchNorm2d) -> Conv2d:
    s, t = _scale_shift(bn)
    out = Conv2d(conv.in_channels, conv.out_channels, conv.kernel_size, conv.stride, conv.padding, conv.dilation,
                 conv.groups, True, conv.padding_mode, dtype=conv.weight.dtype, device=conv.weight.device)
    out.weight.copy_(conv.weight * s.reshape(-1, 1, 1, 1).to(conv.weight.dtype))
    b = conv.bias if conv.bias is not None else torch.zeros_like(s)
    out.bias.copy_((b.to(s.dtype) * s + t).to(conv.weight.dtype))
    return out.eval()


@torch.no_grad()
def FuseLinearBNEval(lin: Linear, bn: BatchNorm1d) -> Linear:
    s, t = _scale_shift(bn)
    out = Linear(lin.in_features, lin.out_features, True, dtype=lin.weight.dtype, device=lin.weight.device)
    out.weight.copy_(lin.weight * s.reshape(-1, 1).to(lin.weight.dtype))
    b = lin.bias if lin.bias is not None else torch.zeros_like(s)
    out.bias.copy_((b.to(s.dtype) * s + t).to(lin.weight.dtype))
    return out.eval()

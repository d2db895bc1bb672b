"""Initialisers (nn/init.go:11-139).  All draw from torch's global generator and
write in place."""
from __future__ import annotations

import math

import torch


def _fans(t: torch.Tensor):
    if t.dim() < 2:
        return t.numel(), t.numel()
    rf = 1
    for s in t.shape[2:]:
        rf *= s
    return t.shape[1] * rf, t.shape[0] * rf


@torch.no_grad()
def Uniform(t, lo: float, hi: float):
    return t.uniform_(lo, hi)


@torch.no_grad()
def Normal(t, mean: float = 0.0, std: float = 1.0):
    return t.normal_(mean, std)


@torch.no_grad()
def Constant(t, v: float):
    return t.fill_(v)


def ZerosInit(t):
    return Constant(t, 0.0)


def OnesInit(t):
    return Constant(t, 1.0)


@torch.no_grad()
def XavierUniform(t, gain: float = 1.0):
    fi, fo = _fans(t)
    a = gain * math.sqrt(6.0 / (fi + fo))
    return t.uniform_(-a, a)


@torch.no_grad()
def XavierNormal(t, gain: float = 1.0):
    fi, fo = _fans(t)
    return t.normal_(0.0, gain * math.sqrt(2.0 / (fi + fo)))


@torch.no_grad()
def KaimingUniform(t, a: float = 0.0):
    fi, _ = _fans(t)
    bound = math.sqrt(2.0 / (1 + a * a)) * math.sqrt(3.0 / fi)
    return t.uniform_(-bound, bound)


@torch.no_grad()
def KaimingNormal(t, a: float = 0.0):
    fi, _ = _fans(t)
    return t.normal_(0.0, math.sqrt(2.0 / (1 + a * a)) / math.sqrt(fi))


@torch.no_grad()
def Orthogonal(t, gain: float = 1.0):
    """Gram-Schmidt on a random normal matrix (rows orthonormal when rows <= cols)."""
    rows = t.shape[0]
    cols = t.numel() // rows
    m = torch.randn(rows, cols, dtype=torch.float64)
    transposed = rows > cols
    if transposed:
        m = m.t().contiguous()
    q = torch.zeros_like(m)
    for i in range(m.shape[0]):
        v = m[i].clone()
        for j in range(i):
            v -= (q[j] @ m[i]) * q[j]
        q[i] = v / v.norm().clamp_min(1e-12)
    if transposed:
        q = q.t()
    t.copy_((gain * q).reshape(t.shape).to(t.dtype))
    return t


@torch.no_grad()
def fan_in_uniform_(weight: torch.Tensor, bias, fan_in: int):
    """The reference's default for Linear / Conv / Bilinear: weight and bias ~ U(-b, b),
    b = sqrt(1 / fan_in), weight drawn first (nn/linear.go:21-33, nn/conv.go:191-211)."""
    b = math.sqrt(1.0 / fan_in)
    # draw in fp32 on the host generator, then cast: the values do not depend on the
    # parameter's dtype or device
    w = torch.empty(weight.shape, dtype=torch.float32).uniform_(-b, b)
    weight.copy_(w.to(weight.dtype))
    if bias is not None:
        bb = torch.empty(bias.shape, dtype=torch.float32).uniform_(-b, b)
        bias.copy_(bb.to(bias.dtype))

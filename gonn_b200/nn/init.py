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


def _resolve_fans(t, fan_in, fan_out):
    """Explicit fans (the reference passes them: nn/init.go:11-41) or the tensor's own."""
    fi, fo = _fans(t)
    return (fi if fan_in is None else int(fan_in)), (fo if fan_out is None else int(fan_out))


@torch.no_grad()
def XavierUniform(t, fan_in=None, fan_out=None, gain: float = 1.0):
    """U(-a, a), a = gain * sqrt(6 / (fan_in + fan_out)); ``XavierUniform(w, fanIn, fanOut)`` as in the
    reference, or ``XavierUniform(w)`` with the fans taken from the shape."""
    fi, fo = _resolve_fans(t, fan_in, fan_out)
    a = gain * math.sqrt(6.0 / (fi + fo))
    return t.uniform_(-a, a)


@torch.no_grad()
def XavierNormal(t, fan_in=None, fan_out=None, gain: float = 1.0):
    fi, fo = _resolve_fans(t, fan_in, fan_out)
    return t.normal_(0.0, gain * math.sqrt(2.0 / (fi + fo)))


@torch.no_grad()
def KaimingUniform(t, fan_in=None, a: float = 0.0):
    """U(-b, b), b = sqrt(2 / (1 + a^2)) * sqrt(3 / fan_in): sqrt(6 / fan_in) at a = 0, the
    reference's bound (nn/init.go:27-33)."""
    fi, _ = _resolve_fans(t, fan_in, None)
    bound = math.sqrt(2.0 / (1 + a * a)) * math.sqrt(3.0 / fi)
    return t.uniform_(-bound, bound)


@torch.no_grad()
def KaimingNormal(t, fan_in=None, a: float = 0.0):
    fi, _ = _resolve_fans(t, fan_in, None)
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

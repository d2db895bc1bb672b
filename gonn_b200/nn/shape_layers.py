"""Padding, resampling, shuffles and distance layers (nn/padding.go, padding_nd.go,
upsample.go, pixel_shuffle.go, shuffle.go, distance.go)."""
from __future__ import annotations

import math

import numpy as np
import torch

from ..ops.window import _src_index, window_gather
from .module import Module

F = torch.nn.functional


def _pad_index(in_shape, pads, mode):
    """Index map of a padded tensor: one tap per output element (-1 = constant fill)."""
    nd = len(in_shape)
    out_shape = tuple(in_shape[d] + pads[d][0] + pads[d][1] for d in range(nd))
    strides = [1] * nd
    for d in range(nd - 2, -1, -1):
        strides[d] = strides[d + 1] * in_shape[d + 1]
    idx = np.zeros((1,), dtype=np.int64)
    valid = np.ones((1,), dtype=bool)
    for d in range(nd):
        src = np.array([_src_index(o - pads[d][0], in_shape[d], mode) for o in range(out_shape[d])])
        idx = (idx[:, None] + (src * strides[d])[None, :]).reshape(-1)
        valid = (valid[:, None] & (src >= 0)[None, :]).reshape(-1)
    return np.where(valid, idx, -1).astype(np.int32)[:, None], out_shape


class _PadNd(Module):
    """Pads the trailing ``nd`` dims.  The amounts are given either as one tuple or as separate
    integers, in the order of the reference's constructors: the 2-D zero / constant /
    reflection / replication layers take ``(top, bottom, left, right)`` (nn/padding.go:28-111);
    the 1-D and 3-D layers and ``CircularPad2d`` take PyTorch's order, last dimension first:
    ``(left, right[, top, bottom[, front, back]])`` (nn/padding_nd.go:155-375).  A single integer
    pads every side alike.  The constant layers take the fill value last (or as ``value=``)."""
    nd, mode = 2, "zeros"
    last_dim_first = False       # argument order: PyTorch's (True) or tensor order (False)
    takes_value = False

    def __init__(self, *padding, value: float = 0.0):
        super().__init__()
        nd = self.nd
        if len(padding) >= 1 and isinstance(padding[0], (tuple, list)):
            if len(padding) == 2 and self.takes_value:
                value = float(padding[1])
            elif len(padding) != 1:
                raise ValueError(f"{type(self).__name__}: unexpected arguments {padding[1:]}")
            padding = tuple(padding[0])
        elif self.takes_value and len(padding) in (2, 2 * nd + 1) and (
                len(padding) != 2 * nd or isinstance(padding[-1], float)):
            padding, value = tuple(padding[:-1]), float(padding[-1])
        if len(padding) == 1:
            padding = (int(padding[0]),) * (2 * nd)
        if len(padding) != 2 * nd:
            raise ValueError(f"{type(self).__name__}: expected {2 * nd} padding values")
        padding = [int(v) for v in padding]
        # stored per dim in tensor order: [(before, after)] for each of the nd trailing dims
        order = range(nd - 1, -1, -1) if self.last_dim_first else range(nd)
        self.pads = [(padding[2 * d], padding[2 * d + 1]) for d in order]
        self.value = value

    def forward(self, x):
        nd = self.nd
        lead = x.shape[:-nd]
        in_shape = tuple(x.shape[-nd:])
        if self.mode == "reflect" and any(max(p) >= s for p, s in zip(self.pads, in_shape)):
            raise ValueError("reflection padding must be smaller than the input size")
        idx, out_shape = _pad_index(in_shape, self.pads, self.mode)
        n = int(np.prod(lead)) if lead else 1
        col = window_gather(x.reshape(n, 1, -1), idx, None, self.value)   # (n, nout, 1)
        return col.reshape(*lead, *out_shape)


class ZeroPad1d(_PadNd):
    """(left, right)."""
    nd, mode, last_dim_first = 1, "zeros", True


class ZeroPad2d(_PadNd):
    """(top, bottom, left, right)."""
    nd, mode = 2, "zeros"


class ZeroPad3d(_PadNd):
    """(left, right, top, bottom, front, back)."""
    nd, mode, last_dim_first = 3, "zeros", True


class ConstantPad1d(_PadNd):
    """(left, right, value)."""
    nd, mode, last_dim_first, takes_value = 1, "zeros", True, True


class ConstantPad2d(_PadNd):
    """(top, bottom, left, right, value)."""
    nd, mode, takes_value = 2, "zeros", True


class ConstantPad3d(_PadNd):
    """(left, right, top, bottom, front, back, value)."""
    nd, mode, last_dim_first, takes_value = 3, "zeros", True, True


class ReflectionPad1d(_PadNd):
    nd, mode, last_dim_first = 1, "reflect", True


class ReflectionPad2d(_PadNd):
    """(top, bottom, left, right)."""
    nd, mode = 2, "reflect"


class ReflectionPad3d(_PadNd):
    nd, mode, last_dim_first = 3, "reflect", True


class ReplicationPad1d(_PadNd):
    nd, mode, last_dim_first = 1, "replicate", True


class ReplicationPad2d(_PadNd):
    """(top, bottom, left, right)."""
    nd, mode = 2, "replicate"


class ReplicationPad3d(_PadNd):
    nd, mode, last_dim_first = 3, "replicate", True


class CircularPad1d(_PadNd):
    nd, mode, last_dim_first = 1, "circular", True


class CircularPad2d(_PadNd):
    """(left, right, top, bottom): PyTorch's order, unlike the other 2-D layers."""
    nd, mode, last_dim_first = 2, "circular", True


class CircularPad3d(_PadNd):
    nd, mode, last_dim_first = 3, "circular", True


def _cubic(t, a=-0.75):
    t = abs(t)
    if t <= 1:
        return (a + 2) * t ** 3 - (a + 3) * t ** 2 + 1
    if t < 2:
        return a * t ** 3 - 5 * a * t ** 2 + 8 * a * t - 4 * a
    return 0.0


def _interp_matrix(n_in, scale, mode, align_corners):
    """(n_out, n_in) constant weight matrix of a 1-D resampling (the reference multiplies by
    such matrices; taps are clamped at the borders)."""
    n_out = n_in * scale
    W = np.zeros((n_out, n_in))
    for o in range(n_out):
        if mode == "nearest":
            W[o, min(o // scale, n_in - 1)] = 1.0
            continue
        if align_corners:
            src = o * (n_in - 1) / (n_out - 1) if n_out > 1 else 0.0
        else:
            src = (o + 0.5) / scale - 0.5
        if mode == "linear":
            src = min(max(src, 0.0), n_in - 1) if not align_corners else src
            i0 = int(math.floor(src))
            f = src - i0
            i1 = min(i0 + 1, n_in - 1)
            i0 = min(max(i0, 0), n_in - 1)
            W[o, i0] += 1 - f
            W[o, i1] += f
        else:  # cubic, Keys kernel a = -0.75, four clamped taps
            i0 = int(math.floor(src))
            f = src - i0
            for k in range(-1, 3):
                W[o, min(max(i0 + k, 0), n_in - 1)] += _cubic(k - f)
    return W


class Upsample(Module):
    """Integer-factor resampling: nearest, linear (1-D), bilinear, bicubic (a = -0.75), trilinear."""

    def __init__(self, scale_factor: int = 2, mode: str = "nearest", align_corners: bool = False):
        super().__init__()
        if int(scale_factor) != scale_factor or scale_factor < 1:
            raise ValueError("Upsample: scale_factor must be a positive integer")
        if mode not in ("nearest", "linear", "bilinear", "bicubic", "trilinear"):
            raise ValueError(f"Upsample: unknown mode {mode!r}")
        self.scale, self.mode, self.align_corners = int(scale_factor), mode, align_corners

    def forward(self, x):
        nd = x.dim() - 2
        want = {"linear": 1, "bilinear": 2, "bicubic": 2, "trilinear": 3}.get(self.mode)
        if want is not None and nd != want:
            raise ValueError(f"Upsample({self.mode}): expected {want} spatial dims, got {nd}")
        kind = {"nearest": "nearest", "bicubic": "cubic"}.get(self.mode, "linear")
        y = x
        for d in range(nd):
            W = torch.from_numpy(_interp_matrix(x.shape[2 + d], self.scale, kind, self.align_corners)).to(
                dtype=x.dtype if x.dtype.is_floating_point else torch.float32, device=x.device)
            y = torch.tensordot(y, W, dims=([2 + d], [1]))        # moves the dim to the end
            y = y.movedim(-1, 2 + d)
        return y


def NewUpsamplingNearest2d(scale_factor: int = 2):
    return Upsample(scale_factor, "nearest")


def NewUpsamplingBilinear2d(scale_factor: int = 2):
    return Upsample(scale_factor, "bilinear", align_corners=True)


UpsamplingNearest2d = NewUpsamplingNearest2d
UpsamplingBilinear2d = NewUpsamplingBilinear2d


class PixelShuffle(Module):
    """(N, C r^2, H, W) -> (N, C, H r, W r): reshape, permute, reshape."""

    def __init__(self, upscale_factor: int):
        super().__init__()
        self.r = upscale_factor

    def forward(self, x):
        N, C, H, W = x.shape
        r = self.r
        if C % (r * r):
            raise ValueError("PixelShuffle: channels must be divisible by r^2")
        return x.reshape(N, C // (r * r), r, r, H, W).permute(0, 1, 4, 2, 5, 3).reshape(N, C // (r * r), H * r, W * r)


class PixelUnshuffle(Module):
    def __init__(self, downscale_factor: int):
        super().__init__()
        self.r = downscale_factor

    def forward(self, x):
        N, C, H, W = x.shape
        r = self.r
        if H % r or W % r:
            raise ValueError("PixelUnshuffle: spatial dims must be divisible by r")
        return x.reshape(N, C, H // r, r, W // r, r).permute(0, 1, 3, 5, 2, 4).reshape(N, C * r * r, H // r, W // r)


class ChannelShuffle(Module):
    def __init__(self, groups: int):
        super().__init__()
        self.groups = groups

    def forward(self, x):
        N, C = x.shape[:2]
        g = self.groups
        if C % g:
            raise ValueError("ChannelShuffle: channels must be divisible by groups")
        return x.reshape(N, g, C // g, *x.shape[2:]).transpose(1, 2).reshape(x.shape)


class CosineSimilarity(Module):
    """sum(x1 x2) / (||x1|| ||x2|| + eps): eps is added to the product of norms, not clamped."""

    def __init__(self, dim: int = 1, eps: float = 1e-8):
        super().__init__()
        self.dim, self.eps = dim, eps

    def forward(self, x1, x2):
        dot = (x1 * x2).sum(self.dim)
        return dot / ((x1 * x1).sum(self.dim).sqrt() * (x2 * x2).sum(self.dim).sqrt() + self.eps)


class PairwiseDistance(Module):
    """(sum |x1 - x2 + eps|^p)^(1/p) over the last dim."""

    def __init__(self, p: float = 2.0, eps: float = 1e-6):
        super().__init__()
        self.p, self.eps = p, eps

    def forward(self, x1, x2):
        return ((x1 - x2 + self.eps).abs() ** self.p).sum(-1) ** (1.0 / self.p)

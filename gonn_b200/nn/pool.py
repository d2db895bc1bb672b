"""Pooling layers (nn/pool.go:18-534, pool_adaptive.go, pool_fractional.go, pool_lp.go,
pool_unpool.go).  Windows come from the same index maps as convolution; the kernels take
the max / mean / LP norm per window directly (the reference gathered windows with a GEMM
and reduced with MaxAxis / MeanAxis)."""
from __future__ import annotations

import math

import numpy as np
import torch

from ..ops.window import _tup, pool as _pool, sliding_index
from .module import Module


class _PoolNd(Module):
    nd, mode = 2, "max"

    def __init__(self, kernel_size, stride=None, padding=0, dilation=1, ceil_mode=False,
                 count_include_pad=True, norm_type: float = 2.0):
        super().__init__()
        nd = self.nd
        self.kernel_size = _tup(kernel_size, nd)
        self.stride = _tup(stride if stride is not None else kernel_size, nd)
        self.padding, self.dilation = _tup(padding, nd), _tup(dilation, nd)
        self.ceil_mode, self.count_include_pad, self.norm_type = ceil_mode, count_include_pad, norm_type

    def _run(self, x):
        if x.dim() != self.nd + 2:
            raise ValueError(f"{type(self).__name__}: expected a {self.nd + 2}-D input")
        N, C = x.shape[:2]
        idx, outs = sliding_index(tuple(x.shape[2:]), self.kernel_size, self.stride, self.padding, self.dilation,
                                  self.ceil_mode)
        y, arg = _pool(x.reshape(N * C, -1), idx, self.mode, self.count_include_pad, self.norm_type)
        if self.mode == "avg" and self.ceil_mode and self.count_include_pad:
            fac = self._overhang_factor(tuple(x.shape[2:]), outs, x.device, y.dtype)
            if fac is not None:
                y = y * fac
        return y.reshape(N, C, *outs), arg, idx, outs

    def _overhang_factor(self, in_shape, outs, device, dtype):
        """Average pooling counts padding cells in its divisor but not the cells a ceil-mode
        window hangs over the padded end (nn/pool.go:264-300): the divisor is the window
        clipped to ``in + 2 * pad``.  The kernel divides by the full window, so windows that
        hang over are rescaled by ``window / clipped``; None when no window does."""
        key = (in_shape, str(device), dtype)
        cache = self.__dict__.setdefault("_fac_cache", {})
        if key not in cache:
            counts = []
            for d in range(self.nd):
                k, st, pad, dil = self.kernel_size[d], self.stride[d], self.padding[d], self.dilation[d]
                lim = in_shape[d] + pad
                counts.append(np.array([sum(1 for j in range(k) if o * st - pad + j * dil < lim)
                                        for o in range(outs[d])], dtype=np.float64))
            div = counts[0]
            for c in counts[1:]:
                div = np.multiply.outer(div, c)
            full = float(np.prod(self.kernel_size))
            fac = full / np.maximum(div.reshape(1, -1), 1.0)
            cache[key] = None if np.all(fac == 1.0) else torch.as_tensor(fac, dtype=dtype, device=device)
        return cache[key]

    def forward(self, x):
        return self._run(x)[0]


class MaxPool1d(_PoolNd):
    nd, mode = 1, "max"

    def ForwardWithIndices(self, x):
        """Returns (y, flat per-plane input index of every maximum)."""
        y, arg, idx, outs = self._run(x)
        N, C = x.shape[:2]
        it = torch.from_numpy(idx.astype(np.int64)).to(x.device)
        flat = it[torch.arange(idx.shape[0], device=x.device)[None], arg.long().clamp_min(0)]
        return y, flat.reshape(N, C, *outs)


class MaxPool2d(MaxPool1d):
    nd = 2


class MaxPool3d(MaxPool1d):
    nd = 3


class AvgPool1d(_PoolNd):
    nd, mode = 1, "avg"


class AvgPool2d(_PoolNd):
    nd, mode = 2, "avg"


class AvgPool3d(_PoolNd):
    nd, mode = 3, "avg"


class LPPool1d(_PoolNd):
    """(sum x^p)^(1/p) per window."""
    nd, mode = 1, "lp"

    def __init__(self, norm_type, kernel_size, stride=None, ceil_mode=False):
        super().__init__(kernel_size, stride, 0, 1, ceil_mode, True, norm_type)


class LPPool2d(LPPool1d):
    nd = 2


class LPPool3d(LPPool1d):
    nd = 3


_adaptive_cache = {}


def _adaptive_index(in_shape, out_shape):
    """Windows [floor(i*in/out), ceil((i+1)*in/out)) per dim, padded with -1 to a common size
    (cached per shape pair: the map depends on nothing else)."""
    key = (tuple(in_shape), tuple(out_shape))
    hit = _adaptive_cache.get(key)
    if hit is None:
        hit = _adaptive_cache[key] = _adaptive_index_build(in_shape, out_shape)
    return hit


def _adaptive_index_build(in_shape, out_shape):
    nd = len(in_shape)
    strides = [1] * nd
    for d in range(nd - 2, -1, -1):
        strides[d] = strides[d + 1] * in_shape[d + 1]
    ranges = [[(i * in_shape[d] // out_shape[d], -(-(i + 1) * in_shape[d] // out_shape[d])) for i in range(out_shape[d])]
              for d in range(nd)]
    wins = []
    import itertools
    for combo in itertools.product(*[range(o) for o in out_shape]):
        axes = [range(*ranges[d][combo[d]]) for d in range(nd)]
        wins.append([sum(c * s for c, s in zip(pt, strides)) for pt in itertools.product(*axes)])
    T = max(len(w) for w in wins)
    idx = np.full((len(wins), T), -1, dtype=np.int32)
    for i, w in enumerate(wins):
        idx[i, :len(w)] = w
    return idx


class _AdaptivePoolNd(Module):
    nd, mode = 2, "avg"

    def __init__(self, *output_size):
        """``AdaptiveAvgPool2d((2, 3))``, ``AdaptiveAvgPool2d(1)`` or, as in the reference,
        ``NewAdaptiveAvgPool2d(2, 3)`` (nn/pool_adaptive.go:95-140)."""
        super().__init__()
        if len(output_size) == 1:
            output_size = output_size[0]
        elif len(output_size) != self.nd:
            raise ValueError(f"{type(self).__name__}: expected 1 or {self.nd} output sizes")
        self.output_size = _tup(output_size, self.nd)

    def forward(self, x):
        N, C = x.shape[:2]
        idx = _adaptive_index(tuple(x.shape[2:]), self.output_size)
        y, _ = _pool(x.reshape(N * C, -1), idx, self.mode, False)
        return y.reshape(N, C, *self.output_size)


class AdaptiveAvgPool1d(_AdaptivePoolNd):
    nd, mode = 1, "avg"


class AdaptiveAvgPool2d(_AdaptivePoolNd):
    nd, mode = 2, "avg"


class AdaptiveAvgPool3d(_AdaptivePoolNd):
    nd, mode = 3, "avg"


class AdaptiveMaxPool1d(_AdaptivePoolNd):
    nd, mode = 1, "max"


class AdaptiveMaxPool2d(_AdaptivePoolNd):
    nd, mode = 2, "max"


class AdaptiveMaxPool3d(_AdaptivePoolNd):
    nd, mode = 3, "max"


class _FractionalMaxPoolNd(Module):
    """Pseudo-random window starts: floor((i+u)*alpha) - floor(u*alpha), alpha = (in-k)/(out-1),
    last start = in - k; one ``u`` per dim per forward (``samples`` fixes them)."""
    nd = 2

    def __init__(self, kernel_size, output_size=None, samples=None, output_ratio=None):
        """Exactly one of ``output_size`` and ``output_ratio`` (output = floor(input * ratio),
        nn/pool_fractional.go:60-110) is given."""
        super().__init__()
        if (output_size is None) == (output_ratio is None):
            raise ValueError(f"{type(self).__name__}: give output_size or output_ratio")
        self.kernel_size = _tup(kernel_size, self.nd)
        self.output_size = _tup(output_size, self.nd) if output_size is not None else None
        self.output_ratio = None
        if output_ratio is not None:
            r = tuple(output_ratio) if isinstance(output_ratio, (tuple, list)) else (output_ratio,) * self.nd
            if len(r) != self.nd or any(not 0 < v <= 1 for v in r):
                raise ValueError(f"{type(self).__name__}: output_ratio needs {self.nd} values in (0, 1]")
            self.output_ratio = r
        self.samples = samples

    def forward(self, x):
        N, C = x.shape[:2]
        in_shape = tuple(x.shape[2:])
        nd = self.nd
        out_size = self.output_size if self.output_size is not None else tuple(
            max(int(math.floor(in_shape[d] * self.output_ratio[d])), 1) for d in range(nd))
        us = self.samples if self.samples is not None else [float(torch.rand(())) for _ in range(nd)]
        starts = []
        for d in range(nd):
            i, k, o = in_shape[d], self.kernel_size[d], out_size[d]
            if k + o - 1 > i:
                raise ValueError("FractionalMaxPool: kernel + output - 1 must not exceed the input size")
            alpha = (i - k) / (o - 1) if o > 1 else 0.0
            st = [int(math.floor((j + us[d]) * alpha) - math.floor(us[d] * alpha)) for j in range(o)]
            st[-1] = i - k
            starts.append(st)
        strides = [1] * nd
        for d in range(nd - 2, -1, -1):
            strides[d] = strides[d + 1] * in_shape[d + 1]
        import itertools
        wins = []
        for combo in itertools.product(*[range(o) for o in out_size]):
            axes = [range(starts[d][combo[d]], starts[d][combo[d]] + self.kernel_size[d]) for d in range(nd)]
            wins.append([sum(c * s for c, s in zip(pt, strides)) for pt in itertools.product(*axes)])
        idx = np.asarray(wins, dtype=np.int32)
        y, _ = _pool(x.reshape(N * C, -1), idx, "max")
        return y.reshape(N, C, *out_size)


class FractionalMaxPool2d(_FractionalMaxPoolNd):
    nd = 2


class FractionalMaxPool3d(_FractionalMaxPoolNd):
    nd = 3


class _MaxUnpoolNd(Module):
    """Scatters values to the flat per-plane indices from ``ForwardWithIndices``; default output
    size (in-1)*stride + kernel; the last write wins on duplicates."""
    nd = 2

    def __init__(self, kernel_size, stride=None):
        super().__init__()
        self.kernel_size = _tup(kernel_size, self.nd)
        self.stride = _tup(stride if stride is not None else kernel_size, self.nd)

    def forward(self, x, indices, output_size=None):
        N, C = x.shape[:2]
        in_sp = tuple(x.shape[2:])
        out_sp = tuple(output_size) if output_size is not None else tuple(
            (in_sp[d] - 1) * self.stride[d] + self.kernel_size[d] for d in range(self.nd))
        S = math.prod(out_sp)
        flat = indices.reshape(N, C, -1).long()
        if bool(((flat < 0) | (flat >= S)).any()):
            raise ValueError("MaxUnpool: index out of range")
        out = torch.zeros(N, C, S, dtype=x.dtype, device=x.device)
        out = out.scatter(2, flat, x.reshape(N, C, -1))
        return out.reshape(N, C, *out_sp)


class MaxUnpool1d(_MaxUnpoolNd):
    nd = 1


class MaxUnpool2d(_MaxUnpoolNd):
    nd = 2


class MaxUnpool3d(_MaxUnpoolNd):
    nd = 3

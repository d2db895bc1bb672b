"""Sliding-window machinery: index maps, im2col / col2im, pooling.

An index map ``idx[win][tap]`` (int32, -1 = padding) describes which input position
each tap of each window reads; it replaces the reference's dense 0/1 gather matrix
(nn/gather.go:23-195).  Maps are built once per geometry on the host and cached.
CUDA tensors use ``csrc/window.cu``; CPU tensors use torch indexing with the same maps.
"""
from __future__ import annotations

import functools
import itertools
from typing import Sequence, Tuple

import numpy as np
import torch

from .. import lib as _l


def _tup(v, n):
    return tuple(v) if isinstance(v, (tuple, list)) else (v,) * n


def out_size(i, k, s, p, d, ceil_mode=False):
    eff = d * (k - 1) + 1
    num = i + 2 * p - eff
    if ceil_mode:
        o = -(-num // s) + 1
        if (o - 1) * s >= i + p:   # last window must start inside the input or left padding
            o -= 1
        return o
    return num // s + 1


def _src_index(pos, size, mode):
    """Maps a (possibly out-of-range) coordinate to a source coordinate for a padding mode."""
    if 0 <= pos < size:
        return pos
    if mode == "zeros":
        return -1
    if mode == "replicate":
        return min(max(pos, 0), size - 1)
    if mode == "circular":
        return pos % size
    if mode == "reflect":
        if size == 1:
            return 0
        period = 2 * (size - 1)
        q = pos % period
        return q if q < size else period - q
    raise ValueError(f"unknown padding mode {mode!r}")


@functools.lru_cache(maxsize=256)
def sliding_index(in_shape: Tuple[int, ...], kernel, stride, padding, dilation, ceil_mode=False,
                  pad_mode="zeros"):
    """Returns (idx [nwin, T] int32 numpy, out_shape)."""
    nd = len(in_shape)
    kernel, stride, padding, dilation = (_tup(v, nd) for v in (kernel, stride, padding, dilation))
    outs = tuple(out_size(in_shape[d], kernel[d], stride[d], padding[d], dilation[d], ceil_mode) for d in range(nd))
    if any(o <= 0 for o in outs):
        raise ValueError(f"sliding window: output size {outs} is not positive")
    strides = [1] * nd
    for d in range(nd - 2, -1, -1):
        strides[d] = strides[d + 1] * in_shape[d + 1]
    per_dim = []
    for d in range(nd):
        o = np.arange(outs[d])[:, None] * stride[d] - padding[d] + np.arange(kernel[d])[None, :] * dilation[d]
        src = np.vectorize(lambda p, sz=in_shape[d]: _src_index(int(p), sz, pad_mode))(o)
        per_dim.append(src)   # [out_d, k_d]
    # combine dims: idx[(o0..), (k0..)]
    idx = np.zeros((1, 1), dtype=np.int64)
    valid = np.ones((1, 1), dtype=bool)
    for d in range(nd):
        src = per_dim[d]
        ow, kw = idx.shape
        idx = (idx[:, None, :, None] + (src * strides[d])[None, :, None, :]).reshape(ow * src.shape[0], kw * src.shape[1])
        valid = (valid[:, None, :, None] & (src >= 0)[None, :, None, :]).reshape(idx.shape)
    idx = np.where(valid, idx, -1).astype(np.int32)
    return idx, outs


@functools.lru_cache(maxsize=256)
def _invert_cached(key, S):
    idx = _MAPS[key]
    flat = idx.reshape(-1)
    pos = np.nonzero(flat >= 0)[0]
    order = np.argsort(flat[pos], kind="stable")
    cols = pos[order].astype(np.int32)
    counts = np.bincount(flat[pos], minlength=S)
    offs = np.zeros(S + 1, dtype=np.int32)
    np.cumsum(counts, out=offs[1:])
    return offs, cols


_MAPS = {}
_DEV = {}


def device_maps(idx: np.ndarray, S: int, device, need_inverse: bool):
    """Device copies of an index map (and its CSR inverse), cached by content."""
    key = (idx.shape, hash(idx.tobytes()), S)
    _MAPS.setdefault(key, idx)
    dk = (key, str(device))
    ent = _DEV.get(dk)
    if ent is None:
        # the kernels trust the map: check its range once, on the host, before it is uploaded
        if idx.size and (int(idx.max()) >= S or int(idx.min()) < -1):
            raise ValueError(f"window index map out of range: values in [{int(idx.min())}, {int(idx.max())}] "
                             f"for a plane of {S} elements (-1 marks padding)")
        ent = {"idx": torch.from_numpy(idx.copy()).to(device)}
        _DEV[dk] = ent
    if need_inverse and "offs" not in ent:
        offs, cols = _invert_cached(key, S)
        ent["offs"] = torch.from_numpy(offs.copy()).to(device)
        ent["cols"] = torch.from_numpy(cols.copy()).to(device)
        # windows that do not overlap (each position in at most one window) get a direct table
        # position -> (window, tap) for the pooling backward, and the windows' valid-tap counts
        counts = np.diff(offs)
        if counts.size and int(counts.max()) <= 1 and S < 2 ** 31:
            T = idx.shape[1]
            p2w = np.zeros((S, 2), dtype=np.int32)
            p2w[:, 0] = -1
            covered = np.nonzero(counts == 1)[0]
            wt = cols[offs[covered]]
            p2w[covered, 0] = wt // T
            p2w[covered, 1] = wt % T
            ent["p2w"] = torch.from_numpy(p2w).to(device)
            ent["wcnt"] = torch.from_numpy((idx >= 0).sum(1).astype(np.int32)).to(device)
    return ent


def _native(x):
    return x.is_cuda and x.dtype in (torch.bfloat16, torch.float16, torch.float32)


def gather_raw(x3, idx_np, kpad, fill=0.0):
    """x3: (N, C, S) -> col (N, nwin, kpad), K = C*T real columns."""
    N, C, S = x3.shape
    nwin, T = idx_np.shape
    if _native(x3):
        m = device_maps(idx_np, S, x3.device, False)
        col = torch.empty((N, nwin, kpad), dtype=x3.dtype, device=x3.device)
        xc = x3.contiguous()
        _l.call("gb_window_gather", _l.I(_l.dtype_code(x3.dtype)), _l.ptr(xc), _l.ptr(m["idx"]), _l.ptr(col),
                _l.I(N), _l.I(C), _l.L(S), _l.I(nwin), _l.I(T), _l.I(kpad), _l.F(fill), _l.stream_ptr())
        return col
    idx = torch.from_numpy(idx_np.astype(np.int64)).to(x3.device)
    safe = idx.clamp_min(0)
    g = x3[:, :, safe.reshape(-1)].reshape(N, C, nwin, T)
    g = torch.where((idx >= 0)[None, None], g, torch.full_like(g, fill))
    col = g.permute(0, 2, 1, 3).reshape(N, nwin, C * T)
    if kpad > C * T:
        col = torch.nn.functional.pad(col, (0, kpad - C * T))
    return col


def scatter_raw(dcol, idx_np, C, S):
    """dcol (N, nwin, kpad) -> dx (N, C, S): the transpose of ``gather_raw``."""
    N, nwin, kpad = dcol.shape
    T = idx_np.shape[1]
    if _native(dcol):
        m = device_maps(idx_np, S, dcol.device, True)
        dx = torch.empty((N, C, S), dtype=dcol.dtype, device=dcol.device)
        dc = dcol.contiguous()
        _l.call("gb_window_scatter", _l.I(_l.dtype_code(dcol.dtype)), _l.ptr(dc), _l.ptr(m["offs"]), _l.ptr(m["cols"]),
                _l.ptr(dx), _l.I(N), _l.I(C), _l.L(S), _l.I(nwin), _l.I(T), _l.I(kpad), _l.I(0), _l.stream_ptr())
        return dx
    idx = torch.from_numpy(idx_np.astype(np.int64)).to(dcol.device)
    g = dcol[:, :, :C * T].reshape(N, nwin, C, T).permute(0, 2, 1, 3).reshape(N, C, nwin * T)
    mask = (idx >= 0).reshape(-1)
    dx = torch.zeros((N, C, S), dtype=dcol.dtype, device=dcol.device)
    dx.index_add_(2, idx.reshape(-1)[mask], g[:, :, mask])
    return dx


class _Gather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x3, idx_np, kpad, fill):
        ctx.meta = (idx_np, x3.shape[1], x3.shape[2])
        return gather_raw(x3, idx_np, kpad, fill)

    @staticmethod
    def backward(ctx, g):
        idx_np, C, S = ctx.meta
        return scatter_raw(g, idx_np, C, S), None, None, None


class _Scatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, dcol, idx_np, C, S):
        ctx.meta = (idx_np, dcol.shape[2])
        return scatter_raw(dcol, idx_np, C, S)

    @staticmethod
    def backward(ctx, g):
        idx_np, kpad = ctx.meta
        return gather_raw(g, idx_np, kpad), None, None, None


def window_gather(x3, idx_np, kpad=None, fill=0.0):
    """Differentiable im2col over a (N, C, S) tensor."""
    C = x3.shape[1]
    kpad = C * idx_np.shape[1] if kpad is None else kpad
    return _Gather.apply(x3, idx_np, kpad, fill)


def window_scatter(dcol, idx_np, C, S):
    """Differentiable col2im (the transpose of ``window_gather``)."""
    return _Scatter.apply(dcol, idx_np, C, S)


_POOL = {"max": 0, "avg": 1, "lp": 2}


class _Pool(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2, idx_np, mode, count_include_pad, p):
        B, S = x2.shape
        nwin, T = idx_np.shape
        m = device_maps(idx_np, S, x2.device, True)
        xc = x2.contiguous()
        y = torch.empty((B, nwin), dtype=x2.dtype, device=x2.device)
        arg = torch.empty((B, nwin), dtype=torch.int32, device=x2.device) if mode == "max" else None
        _l.call("gb_pool_fwd", _l.I(_l.dtype_code(x2.dtype)), _l.ptr(xc), _l.ptr(m["idx"]), _l.ptr(y), _l.ptr(arg),
                _l.L(B), _l.L(S), _l.I(nwin), _l.I(T), _l.I(_POOL[mode]), _l.I(int(count_include_pad)), _l.F(p),
                _l.stream_ptr())
        ctx.save_for_backward(xc, y, arg)
        ctx.meta = (idx_np, mode, count_include_pad, p)
        ctx.mark_non_differentiable(*([] if arg is None else [arg]))
        return (y, arg) if arg is not None else (y, None)

    @staticmethod
    def backward(ctx, dy, _unused=None):
        xc, y, arg = ctx.saved_tensors
        idx_np, mode, cip, p = ctx.meta
        B, S = xc.shape
        nwin, T = idx_np.shape
        m = device_maps(idx_np, S, xc.device, True)
        dx = torch.empty_like(xc)
        dyc = dy.contiguous()
        if "p2w" in m and mode in ("max", "avg"):
            _l.call("gb_pool_bwd_disjoint", _l.I(_l.dtype_code(xc.dtype)), _l.ptr(dyc), _l.ptr(arg), _l.ptr(m["p2w"]),
                    _l.ptr(m["wcnt"]), _l.ptr(dx), _l.L(B), _l.L(S), _l.I(nwin), _l.I(T), _l.I(_POOL[mode]),
                    _l.I(int(cip)), _l.stream_ptr())
            return dx, None, None, None, None
        _l.call("gb_pool_bwd", _l.I(_l.dtype_code(xc.dtype)), _l.ptr(dyc), _l.ptr(xc), _l.ptr(y), _l.ptr(arg),
                _l.ptr(m["idx"]), _l.ptr(m["offs"]), _l.ptr(m["cols"]), _l.ptr(dx), _l.L(B), _l.L(S), _l.I(nwin),
                _l.I(T), _l.I(_POOL[mode]), _l.I(int(cip)), _l.F(p), _l.stream_ptr())
        return dx, None, None, None, None


def pool(x2, idx_np, mode="max", count_include_pad=True, p=2.0):
    """Pools rows of a (B, S) tensor over the windows of ``idx_np``; returns (y, argmax taps)."""
    if _native(x2):
        return _Pool.apply(x2, idx_np, mode, count_include_pad, float(p))
    if x2.is_cuda:
        raise TypeError(f"pool: no CUDA kernel for dtype {x2.dtype}")
    idx = torch.from_numpy(idx_np.astype(np.int64))
    valid = idx >= 0
    g = x2[:, idx.clamp_min(0).reshape(-1)].reshape(x2.shape[0], *idx.shape)
    if mode == "max":
        g = torch.where(valid[None], g, torch.full_like(g, -1e300 if g.dtype == torch.float64 else -3e38))
        y, arg = g.max(-1)
        return y, arg.to(torch.int32)
    if mode == "avg":
        s = torch.where(valid[None], g, torch.zeros_like(g)).sum(-1)
        div = float(idx.shape[1]) if count_include_pad else valid.sum(-1).clamp_min(1).to(g.dtype)[None]
        return s / div, None
    s = torch.where(valid[None], g, torch.zeros_like(g)).pow(p).sum(-1)
    return s.pow(1.0 / p), None

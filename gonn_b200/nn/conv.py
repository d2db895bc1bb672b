"""Convolutions, transposed convolutions, Unfold / Fold (nn/conv.go:17-463, nn/fold.go:45-142).

Forward = im2col by index map (no dense gather matrix) followed by one GEMM per group
against the flattened weight; the output lands directly in (N, C_out, spatial) layout.
Transposed convolution is the adjoint: GEMM then col2im.  Options: stride, padding,
dilation, groups, bias, padding_mode (zeros / reflect / replicate / circular),
output_padding.  Weights and biases ~ U(-b, b), b = sqrt(1 / fan_in), weight first.
"""
from __future__ import annotations

import math

import torch

from ..ops.gemm import gemm
from ..ops.reduce import reduce_axis
from ..ops.window import _tup, sliding_index, window_gather, window_scatter
from ..ops.shape import transpose_last2 as _transpose_last2
from .init import fan_in_uniform_
from .module import Module


class _ConvGemm(torch.autograd.Function):
    """y[n] = W (Co, K) @ col[n]^T (K, L) -> (N, Co, L); trans flags, no transposed copies."""

    @staticmethod
    def forward(ctx, w2, col):
        ctx.save_for_backward(w2, col)
        return gemm(w2, col, trans_b=True)

    @staticmethod
    def backward(ctx, dy):
        w2, col = ctx.saved_tensors
        dy = dy.contiguous()
        dw = dcol = None
        if ctx.needs_input_grad[0]:
            per = gemm(dy, col)                       # (N, Co, K)
            dw = reduce_axis(per, 0, "sum")
        if ctx.needs_input_grad[1]:
            dcol = gemm(dy, w2, trans_a=True)         # (N, L, K)
        return dw, dcol


def _kpad(k, dtype):
    return (k + 7) // 8 * 8 if dtype in (torch.bfloat16, torch.float16) else k


class _ConvNd(Module):
    nd = 2

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1,
                 bias=True, padding_mode="zeros", *, dtype=torch.float32, device=None):
        super().__init__()
        nd = self.nd
        if in_channels % groups or out_channels % groups:
            raise ValueError("conv: channels must be divisible by groups")
        self.in_channels, self.out_channels, self.groups = in_channels, out_channels, groups
        self.kernel_size, self.stride = _tup(kernel_size, nd), _tup(stride, nd)
        self.padding, self.dilation = _tup(padding, nd), _tup(dilation, nd)
        self.padding_mode = padding_mode
        ksz = math.prod(self.kernel_size)
        self.weight = torch.nn.Parameter(torch.empty(out_channels, in_channels // groups, *self.kernel_size,
                                                     dtype=dtype, device=device))
        self.bias = torch.nn.Parameter(torch.empty(out_channels, dtype=dtype, device=device)) if bias else None
        fan_in_uniform_(self.weight.data, self.bias.data if bias else None, (in_channels // groups) * ksz)

    def forward(self, x):
        nd = self.nd
        if x.dim() != nd + 2 or x.shape[1] != self.in_channels:
            raise ValueError(f"{type(self).__name__}: expected (N, {self.in_channels}, ...) with {nd} spatial dims")
        N = x.shape[0]
        spatial = tuple(x.shape[2:])
        idx, outs = sliding_index(spatial, self.kernel_size, self.stride, self.padding, self.dilation, False,
                                  self.padding_mode)
        S = math.prod(spatial)
        G = self.groups
        cg, og = self.in_channels // G, self.out_channels // G
        K = cg * idx.shape[1]
        kp = _kpad(K, x.dtype)
        x3 = x.reshape(N, self.in_channels, S)
        ys = []
        for g in range(G):
            xg = x3 if G == 1 else x3[:, g * cg:(g + 1) * cg]
            col = window_gather(xg, idx, kp)
            w2 = self.weight[g * og:(g + 1) * og].reshape(og, K)
            if kp > K:
                w2 = torch.nn.functional.pad(w2, (0, kp - K))
            ys.append(_ConvGemm.apply(w2, col))
        y = ys[0] if G == 1 else torch.cat(ys, 1)
        if self.bias is not None:
            from ..ops.elementwise import binary
            y = binary("add", y, self.bias.reshape(1, -1, 1))
        return y.reshape(N, self.out_channels, *outs)


class Conv1d(_ConvNd):
    nd = 1


class Conv2d(_ConvNd):
    nd = 2


class Conv3d(_ConvNd):
    nd = 3


class _ConvTransposeNd(Module):
    nd = 2

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, output_padding=0,
                 dilation=1, groups=1, bias=True, *, dtype=torch.float32, device=None):
        super().__init__()
        nd = self.nd
        self.in_channels, self.out_channels, self.groups = in_channels, out_channels, groups
        self.kernel_size, self.stride = _tup(kernel_size, nd), _tup(stride, nd)
        self.padding, self.dilation = _tup(padding, nd), _tup(dilation, nd)
        self.output_padding = _tup(output_padding, nd)
        ksz = math.prod(self.kernel_size)
        self.weight = torch.nn.Parameter(torch.empty(in_channels, out_channels // groups, *self.kernel_size,
                                                     dtype=dtype, device=device))
        self.bias = torch.nn.Parameter(torch.empty(out_channels, dtype=dtype, device=device)) if bias else None
        fan_in_uniform_(self.weight.data, self.bias.data if bias else None, (out_channels // groups) * ksz)

    def forward(self, x):
        nd = self.nd
        N = x.shape[0]
        in_sp = tuple(x.shape[2:])
        out_sp = tuple((in_sp[d] - 1) * self.stride[d] - 2 * self.padding[d] +
                       self.dilation[d] * (self.kernel_size[d] - 1) + self.output_padding[d] + 1 for d in range(nd))
        # the forward conv that maps out_sp -> in_sp defines the windows; we apply its adjoint
        idx, outs = sliding_index(out_sp, self.kernel_size, self.stride, self.padding, self.dilation)
        if tuple(outs) != in_sp:
            raise ValueError("ConvTranspose: inconsistent geometry")
        L, S = math.prod(in_sp), math.prod(out_sp)
        G = self.groups
        cg, og = self.in_channels // G, self.out_channels // G
        T = idx.shape[1]
        K = og * T
        kp = _kpad(K, x.dtype)
        x3 = x.reshape(N, self.in_channels, L)
        ys = []
        for g in range(G):
            xg = (x3 if G == 1 else x3[:, g * cg:(g + 1) * cg])
            w2 = self.weight[g * cg:(g + 1) * cg].reshape(cg, K)          # (Cin_g, Co_g*T)
            if kp > K:
                w2 = torch.nn.functional.pad(w2, (0, kp - K))
            from ..ops.linear import matmul
            dcol = matmul(_transpose_last2(xg), w2)             # (N, L, kp)
            ys.append(window_scatter(dcol, idx, og, S))
        y = ys[0] if G == 1 else torch.cat(ys, 1)
        if self.bias is not None:
            from ..ops.elementwise import binary
            y = binary("add", y, self.bias.reshape(1, -1, 1))
        return y.reshape(N, self.out_channels, *out_sp)


class ConvTranspose1d(_ConvTransposeNd):
    nd = 1


class ConvTranspose2d(_ConvTransposeNd):
    nd = 2


class ConvTranspose3d(_ConvTransposeNd):
    nd = 3


class Unfold(Module):
    """im2col: (N, C, H, W) -> (N, C*kh*kw, L)."""

    def __init__(self, kernel_size, dilation=1, padding=0, stride=1):
        super().__init__()
        self.k, self.d, self.p, self.s = (_tup(v, 2) for v in (kernel_size, dilation, padding, stride))

    def forward(self, x):
        N, C = x.shape[:2]
        idx, _ = sliding_index(tuple(x.shape[2:]), self.k, self.s, self.p, self.d)
        col = window_gather(x.reshape(N, C, -1), idx)
        return col.transpose(1, 2)


class Fold(Module):
    """col2im: (N, C*kh*kw, L) -> (N, C, H, W), overlapping values summed."""

    def __init__(self, output_size, kernel_size, dilation=1, padding=0, stride=1):
        super().__init__()
        self.out = _tup(output_size, 2)
        self.k, self.d, self.p, self.s = (_tup(v, 2) for v in (kernel_size, dilation, padding, stride))

    def forward(self, col):
        N = col.shape[0]
        idx, _ = sliding_index(self.out, self.k, self.s, self.p, self.d)
        T = idx.shape[1]
        C = col.shape[1] // T
        S = self.out[0] * self.out[1]
        return window_scatter(_transpose_last2(col), idx, C, S).reshape(N, C, *self.out)

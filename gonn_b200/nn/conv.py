"""Convolutions, transposed convolutions, Unfold / Fold (nn/conv.go:17-463, nn/fold.go:45-142).

16-bit CUDA tensors with groups = 1 and zero padding run as implicit GEMMs on tcgen05
(csrc/conv.cu): forward, data gradient and weight gradient gather their operands inside the
kernel through the window index map, with the bias in the forward epilogue and the weight
gradient as one GEMM over the whole batch.  Everything else takes the general path:
forward = im2col by index map (no dense gather matrix) followed by one GEMM per group
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


_INV_CACHE = {}


def _inverse_map(idx, S):
    """inv[s][tap] = the window l whose tap `tap` reads position s (idx[l][tap] == s), or -1.
    For zero padding each (s, tap) has at most one such window."""
    import numpy as np
    key = (idx.shape, hash(idx.tobytes()), S)
    inv = _INV_CACHE.get(key)
    if inv is None:
        L, T = idx.shape
        inv = np.full((S, T), -1, dtype=np.int32)
        for t in range(T):
            ls = np.nonzero(idx[:, t] >= 0)[0]
            inv[idx[ls, t], t] = ls
        _INV_CACHE[key] = inv
    return inv


_KTAB_CACHE = {}


def _ktab(C, T, S, device):
    """Device table that splits a contraction index k = c * T + tap into the pair the kernels
    need: {c * S, tap}, padded with {-1, 0} to a multiple of 128 entries."""
    import numpy as np
    key = (C, T, S, str(device))
    t = _KTAB_CACHE.get(key)
    if t is None:
        K = C * T
        n = (K + 127) // 128 * 128
        tab = np.zeros((n, 2), dtype=np.int32)
        tab[:, 0] = -1
        k = np.arange(K)
        tab[:K, 0] = (k // T) * S
        tab[:K, 1] = k % T
        t = torch.from_numpy(tab).to(device)
        _KTAB_CACHE[key] = t
    return t


class _ConvImplicit(torch.autograd.Function):
    """Convolution as implicit GEMMs (csrc/conv.cu): forward, data gradient and weight gradient
    gather their operands inside the kernels; no (N, L, C*T) column tensor exists."""

    @staticmethod
    def forward(ctx, x3, weight, bias, idx, S, L):
        from .. import lib as _l
        from ..ops.window import device_maps
        N, C, _ = x3.shape
        Co = weight.shape[0]
        T = idx.shape[1]
        xc = x3.contiguous()
        wc = weight.contiguous()
        didx = device_maps(idx, S, x3.device, False)["idx"]
        y = torch.empty((N, Co, L), dtype=x3.dtype, device=x3.device)
        if _l.lib().gb_conv_direct_ok(C, T, Co):
            # a contraction of at most 32 (3 channels x 3 x 3): one thread per output position, no tensor-core tile
            _l.call("gb_conv_direct_small", _l.I(_l.dtype_code(x3.dtype)), _l.ptr(xc), _l.ptr(wc), _l.ptr(didx),
                    _l.ptr(bias), _l.ptr(y), _l.I(N), _l.I(C), _l.I(S), _l.I(L), _l.I(T), _l.I(Co), _l.stream_ptr())
        else:
            _l.call("gb_conv_igemm", _l.I(_l.dtype_code(x3.dtype)), _l.ptr(xc), _l.ptr(wc),
                    _l.ptr(_ktab(C, T, S, x3.device)), _l.ptr(didx), _l.ptr(bias), _l.ptr(y), _l.I(N), _l.I(C), _l.I(S),
                    _l.I(L), _l.I(T), _l.I(Co), _l.stream_ptr())
        ctx.save_for_backward(xc, wc)
        ctx.geom = (idx, S, L, T)
        ctx.weight_ref, ctx.bias_ref = weight, bias
        return y

    @staticmethod
    def backward(ctx, dy):
        from .. import lib as _l
        from ..ops.linear import emit_grad
        from ..ops.window import device_maps
        xc, wc = ctx.saved_tensors
        idx, S, L, T = ctx.geom
        N, C, _ = xc.shape
        Co = wc.shape[0]
        dyc = dy.contiguous()
        dt = _l.dtype_code(xc.dtype)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            inv = device_maps(_inverse_map(idx, S), L, xc.device, False)["idx"]
            wt = wc.view(Co, C, T).permute(1, 0, 2).contiguous()        # (C_in, C_out * T)
            dx = torch.empty_like(xc)
            _l.call("gb_conv_igemm", _l.I(dt), _l.ptr(dyc), _l.ptr(wt), _l.ptr(_ktab(Co, T, L, xc.device)), _l.ptr(inv),
                    None, _l.ptr(dx), _l.I(N), _l.I(Co), _l.I(L), _l.I(S), _l.I(T), _l.I(C), _l.stream_ptr())
        if ctx.needs_input_grad[1]:
            didx = device_maps(idx, S, xc.device, False)["idx"]
            splits = int(_l.lib().gb_conv_wgrad_splits(N, L, Co, C, T))
            part = torch.empty(splits * Co * C * T, dtype=torch.float32, device=xc.device)
            w = ctx.weight_ref
            sink = getattr(w, "_gb_sink", None)
            if sink is not None:
                buf, fresh = sink.target(w)
                out, beta = buf, not fresh
            else:
                out, beta = torch.empty(Co * C * T, dtype=xc.dtype, device=xc.device), False
            _l.call("gb_conv_wgrad", _l.I(dt), _l.ptr(xc), _l.ptr(dyc), _l.ptr(_ktab(C, T, S, xc.device)), _l.ptr(didx),
                    _l.ptr(out), _l.ptr(part), _l.I(N), _l.I(C), _l.I(S), _l.I(L), _l.I(T), _l.I(Co), _l.I(int(beta)),
                    _l.stream_ptr())
            if sink is not None:
                sink.ready(w)
            else:
                dw = out.view(w.shape)
        if ctx.bias_ref is not None and ctx.needs_input_grad[2]:
            if Co <= 2048:          # the per-channel partial-sum kernel of BatchNorm, then one add per channel
                from ..ops.batchnorm import lib_ws
                dbt = torch.empty(Co, dtype=dyc.dtype, device=dyc.device)
                _l.call("gb_channel_sum", _l.I(dt), _l.ptr(dyc), _l.ptr(dbt), _l.ptr(lib_ws(Co, dyc.device)), _l.I(N),
                        _l.I(Co), _l.L(L), _l.stream_ptr())
            else:
                per_image = reduce_axis(dyc, 2, "sum", out_dtype=torch.float32)          # (N, Co)
                dbt = reduce_axis(per_image, 0, "sum").to(dyc.dtype)
            db = emit_grad(ctx.bias_ref, dbt)
        return dx, dw, db, None, None, None


def _implicit_ok(x, module):
    import math as _m
    return (x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and module.groups == 1
            and module.padding_mode == "zeros" and module.weight.dtype == x.dtype and x.shape[0] <= 65535
            and _m.prod(module.kernel_size) <= 32 and x[0].numel() < 2 ** 31)


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
        if _implicit_ok(x, self):
            # the parameter itself goes in (its data is (C_out, C_in * T) when read flat), so that the
            # backward finds the gradient sink a data-parallel wrapper may have attached to it
            y = _ConvImplicit.apply(x3, self.weight, self.bias, idx, S, math.prod(outs))
            return y.reshape(N, self.out_channels, *outs)
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

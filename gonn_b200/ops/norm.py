"""LayerNorm / RMSNorm over the last dimension (forward + backward kernels).

Conventions of the reference (nn/norm.go:50-148): biased variance, eps 1e-5 for
LayerNorm and 1e-6 for RMSNorm, RMSNorm(x) = x / sqrt(mean(x^2) + eps) * weight.
"""
from __future__ import annotations

import torch

from .. import lib as _l

_scratch = {}


def _native(x):
    return x.is_cuda and x.dtype in (torch.bfloat16, torch.float16, torch.float32)


def _scratch_for(device, D):
    rows = _l.lib().gb_norm_bwd_scratch_rows()
    key = (device.index, D)
    buf = _scratch.get(key)
    if buf is None:
        buf = torch.empty(rows * 2 * D, dtype=torch.float32, device=device)
        _scratch[key] = buf
    return buf, rows


def norm_ref(x, weight, bias, eps, rms):
    ct = torch.float64 if x.dtype == torch.float64 else torch.float32
    xf = x.to(ct)
    if rms:
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    else:
        mu = xf.mean(-1, keepdim=True)
        var = (xf - mu).pow(2).mean(-1, keepdim=True)
        y = (xf - mu) * torch.rsqrt(var + eps)
    if weight is not None:
        y = y * weight.to(ct)
    if bias is not None and not rms:
        y = y + bias.to(ct)
    return y.to(x.dtype)


def _wdt(x, w):
    if w is None:
        return x.dtype
    if w.dtype not in (x.dtype, torch.float32):
        raise TypeError("norm: weight dtype must equal the input dtype or be float32")
    return w.dtype


class _Norm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps, rms):
        D = x.shape[-1]
        xc = x.contiguous()
        rows = xc.numel() // D
        y = torch.empty_like(xc)
        mean = None if rms else torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        wdt = _wdt(x, weight)
        if bias is not None and bias.dtype != wdt:
            bias = bias.to(wdt)
        _l.call("gb_norm_fwd", _l.I(int(rms)), _l.I(_l.dtype_code(x.dtype)), _l.I(_l.dtype_code(wdt)),
                _l.ptr(xc), _l.ptr(weight), _l.ptr(bias), _l.ptr(y), _l.ptr(mean), _l.ptr(rstd),
                _l.L(rows), _l.I(D), _l.F(eps), _l.stream_ptr())
        ctx.save_for_backward(xc, weight, mean, rstd)
        ctx.rms, ctx.has_bias = rms, bias is not None
        ctx.bias_ref = bias
        return y

    @staticmethod
    def backward(ctx, dy):
        xc, weight, mean, rstd = ctx.saved_tensors
        D = xc.shape[-1]
        rows = xc.numel() // D
        dyc = dy.contiguous()
        dx = torch.empty_like(xc)
        wdt = _wdt(xc, weight)
        need_w = weight is not None and ctx.needs_input_grad[1]
        need_b = ctx.has_bias and ctx.needs_input_grad[2]
        # Parameters owned by a data-parallel wrapper: the reduction kernel writes straight
        # into the gradient bucket on the first write of a step (no accumulation pass, no
        # zero fill); later writes of the same step go through a temporary and are added.
        sunk = []

        def out_for(param, need):
            if not need:
                return None
            sink = getattr(param, "_gb_sink", None)
            if sink is not None and xc.is_cuda:
                buf, fresh = sink.target(param)
                if fresh and buf.dtype == wdt:
                    sunk.append((param, sink, None, None))
                    return buf
                tmp = torch.empty(D, dtype=wdt, device=xc.device)
                sunk.append((param, sink, tmp, buf))
                return tmp
            return torch.empty(D, dtype=wdt, device=xc.device)

        dgamma = out_for(weight, need_w)
        dbeta = out_for(ctx.bias_ref, need_b)
        scratch, srows = _scratch_for(xc.device, D) if (need_w or need_b) else (None, 0)
        _l.call("gb_norm_bwd", _l.I(int(ctx.rms)), _l.I(_l.dtype_code(xc.dtype)), _l.I(_l.dtype_code(wdt)),
                _l.ptr(xc), _l.ptr(dyc), _l.ptr(weight), _l.ptr(mean), _l.ptr(rstd), _l.ptr(dx),
                _l.ptr(dgamma), _l.ptr(dbeta), _l.ptr(scratch), _l.I(srows), _l.L(rows), _l.I(D),
                _l.stream_ptr())
        handled = set()
        for param, sink, tmp, buf in sunk:
            if tmp is not None:
                buf.add_(tmp.to(buf.dtype))
            sink.ready(param)
            handled.add(id(param))
        if weight is not None and id(weight) in handled:
            dgamma = None
        if ctx.bias_ref is not None and id(ctx.bias_ref) in handled:
            dbeta = None
        return dx, dgamma, dbeta, None, None


def layer_norm(x, weight=None, bias=None, eps: float = 1e-5):
    if _native(x):
        return _Norm.apply(x, weight, bias, float(eps), False)
    if x.is_cuda:
        raise TypeError(f"layer_norm: no CUDA kernel for dtype {x.dtype}")
    return norm_ref(x, weight, bias, eps, False)


def rms_norm(x, weight=None, eps: float = 1e-6):
    if _native(x):
        return _Norm.apply(x, weight, None, float(eps), True)
    if x.is_cuda:
        raise TypeError(f"rms_norm: no CUDA kernel for dtype {x.dtype}")
    return norm_ref(x, weight, None, eps, True)

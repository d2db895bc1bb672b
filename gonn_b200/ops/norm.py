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


def _scratch_for(device, D, planes: int = 2):
    rows = _l.lib().gb_norm_bwd_scratch_rows()
    key = (device.index, D, planes)
    buf = _scratch.get(key)
    if buf is None:
        buf = torch.empty(rows * planes * D, dtype=torch.float32, device=device)
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
        need_w = weight is not None and ctx.needs_input_grad[1]
        need_b = ctx.has_bias and ctx.needs_input_grad[2]
        dx, dgamma, dbeta = _norm_backward(ctx, xc, weight, mean, rstd, dy, need_w, need_b)
        return dx, dgamma, dbeta, None, None


class _NormFork(torch.autograd.Function):
    """``(norm(x), x)``: the normalised tensor and the input itself as a second output, for
    blocks of the form ``x + f(norm(x))``.  The gradient of ``x`` is then
    ``norm_bwd(dy) + dpass``; one kernel computes that sum together with the parameter
    gradients and with the column sums of ``dpass``.  Those column sums are the gradient of
    ``res_bias``: the bias of the linear layer whose output (plus the passed-through ``x``)
    forms the next residual stream, ``x + (h W^T + res_bias)``, whose gradient is ``dpass``.
    The caller tells that layer not to compute its bias gradient itself."""

    @staticmethod
    def forward(ctx, x, weight, bias, res_bias, eps, rms):
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
        ctx.rms, ctx.bias_ref, ctx.res_bias = rms, bias, res_bias
        return y, xc.view_as(x)

    @staticmethod
    def backward(ctx, dy, dpass):
        xc, weight, mean, rstd = ctx.saved_tensors
        D = xc.shape[-1]
        rows = xc.numel() // D
        res_bias = ctx.res_bias
        if dy is None or dpass is None or not _fork_shape_ok(xc):
            # one of the two outputs was not used, or rows too wide for the fused kernel:
            # norm backward, sum and column reduction as separate steps
            dx = dgamma = dbeta = None
            if dy is not None:
                dx, dgamma, dbeta = _norm_backward(ctx, xc, weight, mean, rstd, dy, ctx.needs_input_grad[1],
                                                   ctx.bias_ref is not None and ctx.needs_input_grad[2])
            if dpass is not None:
                dx = dpass if dx is None else dx.add_(dpass)
            dsum = None
            if res_bias is not None and ctx.needs_input_grad[3] and dpass is not None:
                from .linear import emit_vector_grad
                dsum = emit_vector_grad(res_bias, dpass.reshape(rows, D))
            return dx, dgamma, dbeta, dsum, None, None
        dyc, dpc = dy.contiguous(), dpass.contiguous()
        dx = torch.empty_like(xc)
        wdt = _wdt(xc, weight)
        need_w = weight is not None and ctx.needs_input_grad[1]
        need_b = ctx.bias_ref is not None and ctx.needs_input_grad[2]
        need_s = res_bias is not None and ctx.needs_input_grad[3]
        outs = _GradOuts(xc.device, D)
        dgamma = outs.take(weight, need_w, wdt)
        dbeta = outs.take(ctx.bias_ref, need_b, wdt)
        # the bias gradient is written in the bias's own dtype when that is the row dtype,
        # otherwise in fp32 and converted below
        s_f32 = need_s and res_bias.dtype != xc.dtype
        dsum, s_acc = outs.take_accumulating(res_bias, need_s, torch.float32 if s_f32 else xc.dtype)
        scratch, srows = _scratch_for(xc.device, D, 3)
        _l.call("gb_norm_bwd_res", _l.I(int(ctx.rms)), _l.I(_l.dtype_code(xc.dtype)), _l.I(_l.dtype_code(wdt)),
                _l.ptr(xc), _l.ptr(dyc), _l.ptr(dpc), _l.ptr(weight), _l.ptr(mean), _l.ptr(rstd), _l.ptr(dx),
                _l.ptr(dgamma), _l.ptr(dbeta), _l.ptr(dsum), _l.I(int(s_f32)), _l.I(int(s_acc)), _l.ptr(scratch),
                _l.I(srows), _l.L(rows), _l.I(D), _l.stream_ptr())
        g = outs.finish({id(weight) if weight is not None else 0: dgamma,
                         id(ctx.bias_ref) if ctx.bias_ref is not None else 1: dbeta,
                         id(res_bias) if res_bias is not None else 2: dsum})
        return (dx, g.get(id(weight)) if weight is not None else None,
                g.get(id(ctx.bias_ref)) if ctx.bias_ref is not None else None,
                g.get(id(res_bias)) if res_bias is not None else None, None, None)


class _GradOuts:
    """Output buffers for small parameter gradients: straight into a data-parallel gradient
    bucket when the parameter has a sink and has not been written this step, a temporary that
    is added afterwards otherwise, a fresh tensor for plain autograd."""

    def __init__(self, device, D):
        self.device, self.D, self.sunk = device, D, []

    def take(self, param, need, dtype):
        if not need:
            return None
        sink = getattr(param, "_gb_sink", None)
        if sink is not None:
            buf, fresh = sink.target(param)
            if fresh and buf.dtype == dtype:
                self.sunk.append((param, sink, None, None))
                return buf
            tmp = torch.empty(self.D, dtype=dtype, device=self.device)
            self.sunk.append((param, sink, tmp, buf))
            return tmp
        return torch.empty(self.D, dtype=dtype, device=self.device)

    def take_accumulating(self, param, need, dtype):
        """Like ``take`` for a kernel that can add into its output: ``(buffer, accumulate)``."""
        if not need:
            return None, False
        sink = getattr(param, "_gb_sink", None)
        if sink is not None:
            buf, fresh = sink.target(param)
            if buf.dtype == dtype:
                self.sunk.append((param, sink, None, None))
                return buf, not fresh
        return self.take(param, need, dtype), False

    def finish(self, by_id):
        """Completes sunk gradients; returns ``{id(param): gradient for autograd}``."""
        done = set()
        for param, sink, tmp, buf in self.sunk:
            if tmp is not None:
                buf.add_(tmp.to(buf.dtype))
            sink.ready(param)
            done.add(id(param))
        out = {}
        for pid, g in by_id.items():
            out[pid] = None if (pid in done or g is None) else g
        return out


def _norm_backward(ctx, xc, weight, mean, rstd, dy, need_w, need_b):
    D = xc.shape[-1]
    rows = xc.numel() // D
    dyc = dy.contiguous()
    dx = torch.empty_like(xc)
    wdt = _wdt(xc, weight)
    outs = _GradOuts(xc.device, D)
    dgamma = outs.take(weight, need_w, wdt)
    dbeta = outs.take(ctx.bias_ref, need_b, wdt)
    scratch, srows = _scratch_for(xc.device, D) if (need_w or need_b) else (None, 0)
    _l.call("gb_norm_bwd", _l.I(int(ctx.rms)), _l.I(_l.dtype_code(xc.dtype)), _l.I(_l.dtype_code(wdt)),
            _l.ptr(xc), _l.ptr(dyc), _l.ptr(weight), _l.ptr(mean), _l.ptr(rstd), _l.ptr(dx),
            _l.ptr(dgamma), _l.ptr(dbeta), _l.ptr(scratch), _l.I(srows), _l.L(rows), _l.I(D),
            _l.stream_ptr())
    g = outs.finish({id(weight) if weight is not None else 0: dgamma,
                     id(ctx.bias_ref) if ctx.bias_ref is not None else 1: dbeta})
    return (dx, g.get(id(weight)) if weight is not None else None,
            g.get(id(ctx.bias_ref)) if ctx.bias_ref is not None else None)


def norm_fork(x, weight=None, bias=None, eps: float = 1e-5, rms: bool = False, res_bias=None):
    """Returns ``(norm(x), x)`` for a residual block ``x + f(norm(x))`` (see ``_NormFork``).
    ``res_bias``: the bias that is added, together with the second output, to form the next
    residual stream; its gradient is then produced here.  Falls back to the plain norm (and
    returns ``x`` unchanged, ``res_bias`` untouched: check ``fork_fuses``) off the fast path."""
    return _NormFork.apply(x, weight, bias, res_bias, float(eps), bool(rms))


def _fork_shape_ok(x) -> bool:
    """Rows of whole 16-byte vectors and at most 8 KB: what the fused backward's ring holds."""
    D = x.shape[-1]
    vec = 4 if x.dtype == torch.float32 else 8
    return D % vec == 0 and D * x.element_size() <= 8192


def fork_fuses(x) -> bool:
    """True when ``norm_fork`` applies to rows like those of ``x`` (native dtypes on CUDA, with
    gradients enabled); rows too wide for the one-kernel backward still work, unfused."""
    return x.is_cuda and x.dtype in (torch.bfloat16, torch.float16, torch.float32) and torch.is_grad_enabled()


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

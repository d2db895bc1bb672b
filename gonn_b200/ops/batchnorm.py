"""BatchNorm forward / backward over (N, C, *) tensors; optional cross-rank statistics.

CUDA: ``csrc/batchnorm.cu`` (statistics exchange fused into the normalise kernels).
CPU: the same formulas with tensor ops; a ``group`` with ``AllReduceSum`` (the TCP group)
provides the cross-rank sums, exactly the packing of distributed/syncbn.go:104-193.
"""
from __future__ import annotations

import torch

from .. import lib as _l


def _native(x):
    return x.is_cuda and x.dtype in (torch.bfloat16, torch.float16, torch.float32)


class _BatchNormTrain(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, running_mean, running_var, eps, momentum, relu, sync):
        N, C = x.shape[:2]
        S = x.numel() // (N * C)
        xc = x.contiguous()
        y = torch.empty_like(xc)
        dev = x.device
        stats = torch.empty(2 * C, dtype=torch.float32, device=dev)
        wf = lib_ws(C, dev)
        w32 = weight.float().contiguous() if weight is not None else None
        b32 = bias.float().contiguous() if bias is not None else None
        slot = sync.slot_offset if sync is not None else 0
        _l.call("gb_bn_fwd", _l.I(_l.dtype_code(x.dtype)), _l.ptr(xc), _l.ptr(y), _l.ptr(w32), _l.ptr(b32),
                _l.ptr(running_mean), _l.ptr(running_var), _l.ptr(stats), _l.ptr(wf), _l.I(N), _l.I(C), _l.L(S),
                _l.F(eps), _l.F(momentum), _l.I(1), _l.I(int(relu)), _l.I(int(sync is not None)), _l.L(slot),
                _l.stream_ptr())
        ctx.save_for_backward(xc, w32, stats, y if relu else None)
        ctx.meta = (N, C, S, relu, sync, weight.dtype if weight is not None else None,
                    bias is not None)
        return y

    @staticmethod
    def backward(ctx, dy):
        xc, w32, stats, y = ctx.saved_tensors
        N, C, S, relu, sync, wdt, has_b = ctx.meta
        dyc = dy.contiguous()
        dx = torch.empty_like(xc)
        dg = torch.empty(C, dtype=torch.float32, device=xc.device)
        db = torch.empty(C, dtype=torch.float32, device=xc.device)
        wf = lib_ws(C, xc.device)
        slot = sync.slot_offset if sync is not None else 0
        _l.call("gb_bn_bwd", _l.I(_l.dtype_code(xc.dtype)), _l.ptr(xc), _l.ptr(dyc), _l.ptr(dx), _l.ptr(w32),
                _l.ptr(stats), _l.ptr(dg), _l.ptr(db), _l.ptr(wf), _l.I(N), _l.I(C), _l.L(S),
                _l.I(int(sync is not None)), _l.L(slot), _l.ptr(y if relu else None), _l.stream_ptr())
        return (dx, dg.to(wdt) if wdt is not None else None, db.to(wdt) if has_b else None,
                None, None, None, None, None, None)


_ws_cache = {}


def lib_ws(C, dev):
    """Scratch of one BatchNorm call (partial sums, the finalised sums, the ready flag and the
    election word), kept per (device, stream, C) and zeroed once: calls on one stream run in
    order, and the flag words only ever hold serial numbers, which start at 1."""
    key = (dev.index, _l.current_stream_handle(), C)
    buf = _ws_cache.get(key)
    if buf is None:
        f = _l.lib().gb_bn_workspace_floats
        f.restype = _l.L
        buf = torch.zeros(int(f(_l.I(C))), dtype=torch.float32, device=dev)
        _ws_cache[key] = buf
    return buf


def batch_norm_eval(x, weight, bias, running_mean, running_var, eps, relu=False):
    if _native(x):
        N, C = x.shape[:2]
        S = x.numel() // (N * C)
        xc = x.contiguous()
        y = torch.empty_like(xc)
        w32 = weight.detach().float().contiguous() if weight is not None else None
        b32 = bias.detach().float().contiguous() if bias is not None else None
        _l.call("gb_bn_fwd", _l.I(_l.dtype_code(x.dtype)), _l.ptr(xc), _l.ptr(y), _l.ptr(w32), _l.ptr(b32),
                _l.ptr(running_mean), _l.ptr(running_var), None, None, _l.I(N), _l.I(C), _l.L(S), _l.F(eps),
                _l.F(0.0), _l.I(0), _l.I(int(relu)), _l.I(0), _l.L(0), _l.stream_ptr())
        return y
    shape = [1, -1] + [1] * (x.dim() - 2)
    y = (x - running_mean.reshape(shape).to(x.dtype)) * torch.rsqrt(running_var.reshape(shape).to(x.dtype) + eps)
    if weight is not None:
        y = y * weight.reshape(shape)
    if bias is not None:
        y = y + bias.reshape(shape)
    return torch.relu(y) if relu else y


def batch_norm_train(x, weight, bias, running_mean, running_var, eps=1e-5, momentum=0.1, relu=False,
                     sync=None, group=None):
    """Training forward.  ``sync``: a device-side exchange (``distributed.syncbn.DeviceSync``);
    ``group``: a host group with ``AllReduceSum`` (CPU ranks).  Running statistics (fp32
    buffers) are updated in place from the global statistics."""
    if _native(x) and group is None:
        return _BatchNormTrain.apply(x, weight, bias, running_mean, running_var, float(eps), float(momentum),
                                     bool(relu), sync)
    # host formulas (also the oracle): sums -> (all-reduce) -> mean / var -> normalise
    N, C = x.shape[:2]
    dims = [0] + list(range(2, x.dim()))
    shape = [1, C] + [1] * (x.dim() - 2)
    ct = torch.float64 if x.dtype == torch.float64 else torch.float32
    xf = x.to(ct)
    count = torch.tensor([x.numel() / C], dtype=ct)
    if group is not None and group.WorldSize() > 1:
        packed = torch.cat([xf.sum(dims).detach(), (xf * xf).sum(dims).detach(), count]).double()
        return _HostSyncBN.apply(x, weight, bias, running_mean, running_var, eps, momentum, group, relu)
    mean = xf.mean(dims)
    var = (xf * xf).mean(dims) - mean * mean if False else xf.var(dims, unbiased=False)
    n = float(count)
    with torch.no_grad():
        if running_mean is not None:
            running_mean.mul_(1 - momentum).add_(momentum * mean.detach().to(running_mean.dtype))
            unb = var.detach() * n / (n - 1) if n > 1 else var.detach()
            running_var.mul_(1 - momentum).add_(momentum * unb.to(running_var.dtype))
    y = (xf - mean.reshape(shape)) * torch.rsqrt(var.reshape(shape) + eps)
    if weight is not None:
        y = y * weight.reshape(shape).to(ct)
    if bias is not None:
        y = y + bias.reshape(shape).to(ct)
    y = y.to(x.dtype)
    return torch.relu(y) if relu else y


class _HostSyncBN(torch.autograd.Function):
    """SyncBatchNorm on host ranks: [sum x | sum x^2 | n] all-reduced in forward,
    [sum dy | sum dy*xhat] in backward; dgamma / dbeta keep the LOCAL sums."""

    @staticmethod
    def forward(ctx, x, weight, bias, running_mean, running_var, eps, momentum, group, relu):
        C = x.shape[1]
        dims = [0] + list(range(2, x.dim()))
        shape = [1, C] + [1] * (x.dim() - 2)
        xf = x.double()
        packed = torch.cat([xf.sum(dims), (xf * xf).sum(dims), torch.tensor([x.numel() / C], dtype=torch.float64)])
        group.AllReduceSum(packed)
        n = float(packed[-1])
        mean = packed[:C] / n
        var = (packed[C:2 * C] / n - mean * mean).clamp_min(0)
        invstd = torch.rsqrt(var + eps)
        if running_mean is not None:
            running_mean.mul_(1 - momentum).add_(momentum * mean.to(running_mean.dtype))
            unb = var * n / (n - 1) if n > 1 else var
            running_var.mul_(1 - momentum).add_(momentum * unb.to(running_var.dtype))
        xh = (xf - mean.reshape(shape)) * invstd.reshape(shape)
        y = xh
        if weight is not None:
            y = y * weight.double().reshape(shape)
        if bias is not None:
            y = y + bias.double().reshape(shape)
        if relu:
            y = torch.relu(y)
        ctx.save_for_backward(xh, weight, invstd, y if relu else None)
        ctx.meta = (group, n, dims, shape, relu, bias is not None)
        return y.to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        xh, weight, invstd, y = ctx.saved_tensors
        group, n, dims, shape, relu, has_b = ctx.meta
        C = xh.shape[1]
        g = dy.double()
        if relu:
            g = g * (y > 0)
        s1, s2 = g.sum(dims), (g * xh).sum(dims)
        dbeta, dgamma = s1.clone(), s2.clone()       # local copies, before the in-place reduce
        red = torch.cat([s1, s2])
        group.AllReduceSum(red)
        m1, m2 = red[:C] / n, red[C:] / n
        dx = invstd.reshape(shape) * (g - m1.reshape(shape) - xh * m2.reshape(shape))
        if weight is not None:
            dx = dx * weight.double().reshape(shape)
        return (dx.to(dy.dtype), dgamma.to(weight.dtype) if weight is not None else None,
                dbeta.to(weight.dtype) if has_b else None, None, None, None, None, None, None)

"""Softmax / log-softmax over an axis and fused cross-entropy.

CUDA: ``csrc/softmax_ce.cu``.  CPU: torch expressions with the same semantics
(reference: tensor/ops_activation.go:454-470, nn/loss.go:131-242 — class weights,
ignore index, label smoothing; the mean divides by the summed weights of the
non-ignored targets).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import lib as _l


def _native(x):
    return x.is_cuda and x.dtype in (torch.bfloat16, torch.float16, torch.float32)


class _Softmax(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, log):
        D = x.shape[-1]
        xc = x.contiguous()
        y = torch.empty_like(xc)
        _l.call("gb_softmax_fwd", _l.I(int(log)), _l.I(_l.dtype_code(x.dtype)), _l.ptr(xc), _l.ptr(y),
                _l.L(xc.numel() // D), _l.I(D), _l.stream_ptr())
        ctx.save_for_backward(y)
        ctx.log = log
        return y

    @staticmethod
    def backward(ctx, dy):
        (y,) = ctx.saved_tensors
        D = y.shape[-1]
        dyc = dy.contiguous()
        dx = torch.empty_like(y)
        _l.call("gb_softmax_bwd", _l.I(int(ctx.log)), _l.I(_l.dtype_code(y.dtype)), _l.ptr(y), _l.ptr(dyc),
                _l.ptr(dx), _l.L(y.numel() // D), _l.I(D), _l.stream_ptr())
        return dx, None


def _softmax_any(x, axis, log):
    axis = axis % x.dim()
    if not _native(x):
        if x.is_cuda and x.dtype != torch.float64:
            raise TypeError(f"softmax: no CUDA kernel for dtype {x.dtype}")
        return torch.log_softmax(x, axis) if log else torch.softmax(x, axis)
    if axis != x.dim() - 1:
        return _Softmax.apply(x.transpose(axis, -1).contiguous(), log).transpose(axis, -1)
    return _Softmax.apply(x, log)


def softmax(x, axis: int = -1):
    return _softmax_any(x, axis, False)


def log_softmax(x, axis: int = -1):
    return _softmax_any(x, axis, True)


def cross_entropy_ref(logits, targets, weight=None, ignore_index=None, label_smoothing=0.0,
                      reduction="mean"):
    """Oracle: the reference's decomposition, evaluated in fp32/fp64 with torch."""
    ct = torch.float64 if logits.dtype == torch.float64 else torch.float32
    logp = torch.log_softmax(logits.to(ct), dim=1)
    N, C = logp.shape
    t = targets.long()
    keep = torch.ones(N, dtype=ct, device=logits.device)
    if ignore_index is not None:
        keep = (t != ignore_index).to(ct)
    safe = torch.where(keep.bool(), t, torch.zeros_like(t))
    w = keep if weight is None else weight.to(ct)[safe] * keep
    vec = -logp.gather(1, safe[:, None]).squeeze(1) * w
    denom = w.sum()
    if label_smoothing:
        smooth = -(logp * (weight.to(ct)[None, :] if weight is not None else 1.0)).sum(1) * keep
        vec = vec * (1 - label_smoothing) + smooth * (label_smoothing / C)
    if reduction == "sum":
        return vec.sum()
    if reduction == "none":
        return vec
    return vec.sum() / denom


class _CrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, weight, ignore_index, eps, reduction, inplace):
        N, C = logits.shape
        xc = logits.contiguous()
        t = targets.to(torch.int64).contiguous()
        dev = logits.device
        loss_row = torch.empty(N, dtype=torch.float32, device=dev)
        lse = torch.empty(N, dtype=torch.float32, device=dev)
        w_row = torch.empty(N, dtype=torch.float32, device=dev)
        out2 = torch.empty(2, dtype=torch.float32, device=dev)
        cw = weight.to(torch.float32).contiguous() if weight is not None else None
        cw_sum = float(cw.sum().item()) if cw is not None else float(C)
        red = {"mean": 0, "sum": 1, "none": 2}[reduction]
        _l.call("gb_ce_fwd", _l.I(_l.dtype_code(xc.dtype)), _l.ptr(xc), _l.ptr(t), _l.ptr(cw), _l.F(cw_sum),
                _l.ptr(loss_row), _l.ptr(lse), _l.ptr(w_row), _l.ptr(out2), _l.L(N), _l.I(C),
                _l.L(ignore_index if ignore_index is not None else 0), _l.I(int(ignore_index is not None)),
                _l.F(eps), _l.I(red), _l.stream_ptr())
        ctx.save_for_backward(xc, t, cw, lse, out2)
        ctx.meta = (ignore_index, eps, reduction, cw_sum, inplace)
        if reduction == "none":
            return loss_row
        return out2[0]

    @staticmethod
    def backward(ctx, g):
        xc, t, cw, lse, out2 = ctx.saved_tensors
        ignore_index, eps, reduction, cw_sum, inplace = ctx.meta
        N, C = xc.shape
        dx = xc if inplace else torch.empty_like(xc)
        g = g.to(torch.float32).contiguous()
        g_scalar = g if reduction != "none" else None
        g_row = g if reduction == "none" else None
        denom = out2[1:] if reduction == "mean" else None
        _l.call("gb_ce_bwd", _l.I(_l.dtype_code(xc.dtype)), _l.ptr(xc), _l.ptr(t), _l.ptr(cw), _l.F(cw_sum),
                _l.ptr(lse), _l.ptr(g_scalar), _l.ptr(g_row), _l.ptr(denom), _l.ptr(dx), _l.L(N), _l.I(C),
                _l.L(ignore_index if ignore_index is not None else 0), _l.I(int(ignore_index is not None)),
                _l.F(eps), _l.stream_ptr())
        return dx, None, None, None, None, None, None


class _CrossEntropyFused(torch.autograd.Function):
    """Loss and gradient in one kernel: the forward leaves ``softmax - onehot`` (already divided by N
    for the mean) in the logits' buffer, the backward multiplies it by the upstream scalar with a
    kernel that returns at once when that scalar is 1."""

    @staticmethod
    def forward(ctx, logits, targets, reduction):
        N, C = logits.shape
        t = targets.to(torch.int64).contiguous()
        dev = logits.device
        loss_row = torch.empty(N, dtype=torch.float32, device=dev)
        w_row = torch.empty(N, dtype=torch.float32, device=dev)
        out2 = torch.empty(2, dtype=torch.float32, device=dev)
        _l.call("gb_ce_fused", _l.I(_l.dtype_code(logits.dtype)), _l.ptr(logits), _l.ptr(t), _l.ptr(loss_row),
                _l.ptr(w_row), _l.ptr(out2), _l.L(N), _l.I(C), _l.I({"mean": 0, "sum": 1}[reduction]),
                _l.stream_ptr())
        ctx.grad_buf = logits          # holds the gradient now
        return out2[0]

    @staticmethod
    def backward(ctx, g):
        dx = ctx.grad_buf
        g = g.to(torch.float32).contiguous()
        _l.call("gb_scale_unless_one", _l.I(_l.dtype_code(dx.dtype)), _l.ptr(dx), _l.L(dx.numel()), _l.ptr(g),
                _l.stream_ptr())
        return dx, None, None


def _fused_ok(logits, weight, ignore_index, label_smoothing, reduction) -> bool:
    return (logits.dtype in (torch.bfloat16, torch.float16) and logits.is_contiguous() and logits.shape[1] % 8 == 0
            and logits.data_ptr() % 16 == 0 and weight is None and ignore_index is None
            and label_smoothing == 0.0 and reduction in ("mean", "sum") and logits.requires_grad
            and torch.is_grad_enabled())


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor, weight: Optional[torch.Tensor] = None,
                  ignore_index: Optional[int] = None, label_smoothing: float = 0.0,
                  reduction: str = "mean", inplace_backward: bool = False,
                  consume_logits: bool = False) -> torch.Tensor:
    """Cross-entropy over (N, C) logits and (N,) class indices.

    ``inplace_backward`` lets the backward kernel write the logits' gradient over
    the logits buffer (valid when nothing else reads the logits after the backward pass).
    ``consume_logits`` goes further: the logits are gone when this call returns, because
    the forward kernel already writes the gradient over them (one pass over the logits
    instead of two; for models whose loss is computed inside the model and whose logits
    nobody else sees).  It applies to 16-bit logits with a class count that is a multiple
    of 8, no class weights, ignored index or label smoothing; other calls ignore the flag.
    """
    if logits.dim() != 2:
        raise ValueError("cross_entropy: logits must be (N, C)")
    if _native(logits) and consume_logits and _fused_ok(logits, weight, ignore_index, label_smoothing, reduction):
        return _CrossEntropyFused.apply(logits, targets, reduction)
    if _native(logits):
        return _CrossEntropy.apply(logits, targets, weight, ignore_index, float(label_smoothing),
                                   reduction, bool(inplace_backward))
    if logits.is_cuda and logits.dtype != torch.float64:
        raise TypeError(f"cross_entropy: no CUDA kernel for dtype {logits.dtype}")
    return cross_entropy_ref(logits, targets, weight, ignore_index, label_smoothing, reduction)

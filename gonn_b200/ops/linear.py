"""Linear layer math with fused epilogues: ``y = act(x W^T + b)``.

Forward is one GEMM (bias and activation in its epilogue, pre-activation saved
by the same epilogue when an activation is present).  Backward is two GEMMs that
use the trans flags instead of transposed copies (data gradient ``dy W``, weight
gradient ``dy^T x``) plus a column reduction for the bias.  The reference builds
the same three products from MatMul/Transpose/Add tape nodes (nn/linear.go:40-59,
tensor/ops_matmul.go:29-46) and copies W on every forward.

Gradient sinks: when a parameter carries a ``_gb_sink`` attribute (installed by
the data-parallel wrappers), its gradient is written straight into the sink's
flat bucket (overwrite on the first write of a step, accumulate afterwards) and
``None`` is returned to autograd, so no separate accumulation pass runs.

Ordering rule for every op that uses a sink: ``sink.ready(p)`` may launch the bucket's
fused optimizer step on another stream, which rewrites ``p`` in place.  An op must
therefore issue every kernel that reads ``p`` (the data-gradient GEMM reads the weight)
before it calls ``emit_*`` for ``p``; the sink orders its launch after the kernels
already issued on the compute stream.
"""
from __future__ import annotations

from typing import Optional

import torch

from .elementwise import unary_backward
from .gemm import gemm
from .reduce import column_sum

_DACT_MODE = {"relu": "mul_drelu", "gelu": "mul_dgelu", "gelu_tanh": "mul_dgelu",
              "geluexact": "mul_dgeluexact", "gelu_erf": "mul_dgeluexact"}
_ACT_UNARY = {"relu": "relu", "gelu": "gelu", "gelu_tanh": "gelu", "geluexact": "geluexact",
              "gelu_erf": "geluexact"}


def emit_weight_grad(param: torch.Tensor, a: torch.Tensor, b: torch.Tensor, trans_a: bool,
                     trans_b: bool):
    """Computes op(a) @ op(b) as the gradient of ``param``; honours a gradient sink."""
    sink = getattr(param, "_gb_sink", None)
    if sink is not None:
        buf, fresh = sink.target(param)
        gemm(a, b, trans_a=trans_a, trans_b=trans_b, out=buf.view(param.shape), beta=not fresh)
        sink.ready(param)
        return None
    return gemm(a, b, trans_a=trans_a, trans_b=trans_b, out_dtype=param.dtype)


def emit_vector_grad(param: torch.Tensor, rows2d: torch.Tensor):
    """Column sum of ``rows2d`` as the gradient of a bias-like ``param``."""
    sink = getattr(param, "_gb_sink", None)
    if sink is not None:
        buf, fresh = sink.target(param)
        column_sum(rows2d, out=buf.view(param.shape), accumulate=not fresh)
        sink.ready(param)
        return None
    return column_sum(rows2d, out_dtype=param.dtype)


def emit_grad(param: torch.Tensor, grad: torch.Tensor):
    """Hands an already computed gradient to the sink (copy or add) or back to autograd."""
    sink = getattr(param, "_gb_sink", None)
    if sink is not None:
        buf, fresh = sink.target(param)
        v = buf.view(param.shape)
        if fresh:
            v.copy_(grad)
        else:
            v.add_(grad)
        sink.ready(param)
        return None
    return grad


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, act, residual, bias_grad=True):
        K = x.shape[-1]
        N = weight.shape[0]
        x2 = x.reshape(-1, K)
        pre = None
        aux, aux_mode = None, None
        if act is not None and act != "none":
            pre = torch.empty((x2.shape[0], N), dtype=x.dtype, device=x.device)
            aux, aux_mode = pre, "store_pre"
            if residual is not None:
                raise ValueError("linear: activation and residual cannot be combined")
        elif residual is not None:
            aux, aux_mode = residual.reshape(-1, N), "add"
        y = gemm(x2, weight, trans_b=True, bias=bias, act=act, aux=aux, aux_mode=aux_mode)
        ctx.save_for_backward(x2, weight, pre)
        ctx.act, ctx.has_bias, ctx.xshape = act, bias is not None, x.shape
        ctx.bias_ref = bias
        ctx.has_res = residual is not None
        ctx.bias_grad = bias_grad
        return y.reshape(*x.shape[:-1], N)

    @staticmethod
    def backward(ctx, dy):
        x2, weight, pre = ctx.saved_tensors
        N = weight.shape[0]
        dy2 = dy.reshape(-1, N)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dres = dy if ctx.has_res else None
        if pre is not None:
            dy2 = unary_backward(_ACT_UNARY[ctx.act], pre, dy2)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, weight).reshape(ctx.xshape)
        if ctx.needs_input_grad[1]:
            dw = emit_weight_grad(weight, dy2, x2, True, False)
        if ctx.has_bias and ctx.needs_input_grad[2] and ctx.bias_grad:
            db = emit_vector_grad(ctx.bias_ref, dy2)
        return dx, dw, db, None, dres, None


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           act: Optional[str] = None, residual: Optional[torch.Tensor] = None,
           bias_grad: bool = True) -> torch.Tensor:
    """``act(x @ weight.T + bias)`` (+ ``residual`` when no activation); weight is (out, in).
    ``bias_grad=False``: the bias gradient is produced elsewhere (``ops.norm.norm_fork`` yields
    it from the residual stream's gradient), so the column reduction is skipped here."""
    return _Linear.apply(x, weight, bias, act, residual, bias_grad)


class _FeedForward(torch.autograd.Function):
    """``act(x W1^T + b1) W2^T + b2 (+ residual)`` as one tape node.

    Keeping both products in one node lets the backward fold the activation's derivative
    into the epilogue of the data-gradient GEMM of the second layer
    (``dpre = (dy W2) * act'(pre)``), so no separate elementwise pass over the hidden
    activations runs in either direction.
    """

    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2, act, residual, bias2_grad=True):
        K, F, N = x.shape[-1], w1.shape[0], w2.shape[0]
        x2 = x.reshape(-1, K)
        pre = torch.empty((x2.shape[0], F), dtype=x.dtype, device=x.device)
        h = gemm(x2, w1, trans_b=True, bias=b1, act=act, aux=pre, aux_mode="store_pre")
        res2 = residual.reshape(-1, N) if residual is not None else None
        y = gemm(h, w2, trans_b=True, bias=b2, aux=res2, aux_mode="add" if res2 is not None else None)
        ctx.save_for_backward(x2, w1, w2, pre, h)
        ctx.act, ctx.xshape, ctx.has_res = act, x.shape, residual is not None
        ctx.b1, ctx.b2 = b1, b2
        ctx.bias2_grad = bias2_grad
        return y.reshape(*x.shape[:-1], N)

    @staticmethod
    def backward(ctx, dy):
        x2, w1, w2, pre, h = ctx.saved_tensors
        N = w2.shape[0]
        dy2 = dy.reshape(-1, N)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dres = dy if ctx.has_res else None
        # every read of a weight comes before its gradient is declared ready (module docstring):
        # second layer's data gradient (act' folded in) first, then its weight / bias gradients
        dpre = gemm(dy2, w2, aux=pre, aux_mode=_DACT_MODE[ctx.act])
        dw2 = emit_weight_grad(w2, dy2, h, True, False) if ctx.needs_input_grad[3] else None
        db2 = (emit_vector_grad(ctx.b2, dy2)
               if (ctx.b2 is not None and ctx.needs_input_grad[4] and ctx.bias2_grad) else None)
        dx = gemm(dpre, w1).reshape(ctx.xshape) if ctx.needs_input_grad[0] else None
        dw1 = emit_weight_grad(w1, dpre, x2, True, False) if ctx.needs_input_grad[1] else None
        db1 = emit_vector_grad(ctx.b1, dpre) if (ctx.b1 is not None and ctx.needs_input_grad[2]) else None
        return dx, dw1, db1, dw2, db2, None, dres, None


def feed_forward(x, w1, b1, w2, b2, act: str = "gelu", residual: Optional[torch.Tensor] = None,
                 bias2_grad: bool = True):
    """Two-layer feed-forward block with a fusable activation (relu / gelu / geluexact).
    ``bias2_grad=False``: see ``linear``."""
    if act not in _DACT_MODE:
        raise ValueError(f"feed_forward: activation {act!r} cannot be fused")
    return _FeedForward.apply(x, w1, b1, w2, b2, act, residual, bias2_grad)


class _MatMul(torch.autograd.Function):
    """C = A @ B for 2-D / batched operands; backward via trans flags (no transposes)."""

    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        return gemm(a, b)

    @staticmethod
    def backward(ctx, g):
        a, b = ctx.saved_tensors
        g = g.contiguous()
        da = db = None
        if ctx.needs_input_grad[0]:
            da = gemm(g, b, trans_b=True)
            if a.dim() == 2 and da.dim() == 3:
                da = da.sum(0)
        if ctx.needs_input_grad[1]:
            db = gemm(a, g, trans_a=True)
            if b.dim() == 2 and db.dim() == 3:
                db = db.sum(0)
        return da, db


def matmul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Differentiable matrix product with NumPy-style batch broadcasting (rank <= 3 on the
    kernel path; higher ranks are flattened into one batch dimension)."""
    if a.dim() == 1 or b.dim() == 1:
        a2 = a[None, :] if a.dim() == 1 else a
        b2 = b[:, None] if b.dim() == 1 else b
        r = matmul(a2, b2)
        if a.dim() == 1:
            r = r.squeeze(-2)
        if b.dim() == 1:
            r = r.squeeze(-1)
        return r
    if a.dim() > 3 or b.dim() > 3:
        bs = torch.broadcast_shapes(a.shape[:-2], b.shape[:-2])
        a3 = a.expand(*bs, *a.shape[-2:]).reshape(-1, *a.shape[-2:])
        b3 = b.expand(*bs, *b.shape[-2:]).reshape(-1, *b.shape[-2:])
        return _MatMul.apply(a3, b3).reshape(*bs, a.shape[-2], b.shape[-1])
    if not ((a.requires_grad or b.requires_grad) and torch.is_grad_enabled()):
        return gemm(a, b)                     # nothing to record: skip the tape node
    return _MatMul.apply(a, b)

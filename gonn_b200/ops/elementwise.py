"""Elementwise ops: the unary registry's kernels (forward and backward), binary ops
with broadcasting, casts.

Every op has two evaluation paths with the same formulas: the CUDA kernels in
``csrc/elementwise.cu`` for CUDA tensors, and a torch expression for CPU tensors
(the oracle path).  The op list and the formulas follow the reference's registry
(tensor/ops_unary.go:12-138, tensor/ops_activation.go:17-450); GELU is the tanh
approximation, ``geluexact`` the erf form, softplus is linear above 20.
"""
from __future__ import annotations

import math
from typing import Callable, Dict, Tuple

import torch

from .. import lib as _l

# op ids: keep in sync with csrc/elementwise.cu
UNARY_IDS = {name: i for i, name in enumerate([
    "exp", "log", "sqrt", "sin", "cos", "tan", "abs", "reciprocal", "square",
    "relu", "selu", "sigmoid", "tanh", "hardtanh", "hardsigmoid", "softplus", "softsign",
    "gelu", "geluexact", "silu", "hardswish", "mish", "relu6", "logsigmoid", "tanhshrink",
    "pow", "clip", "leakyrelu", "elu", "hardshrink", "softshrink", "softplusbeta", "threshold",
    "celu", "neg", "scale_add"])}
BINARY_IDS = {"add": 0, "sub": 1, "mul": 2, "div": 3}
REGISTERED_UNARY = [n for n, i in UNARY_IDS.items() if i < 25]  # the 25 parameter-free names

_SELU_A, _SELU_S = 1.6732632423543772848170429916717, 1.0507009873554804934193349852946
_K0, _K1 = 0.7978845608028654, 0.044715
F = torch.nn.functional


def _sp(x):  # softplus, linear above 20
    return torch.where(x > 20, x, torch.log1p(torch.exp(torch.clamp(x, max=20.0))))


# name -> (forward(x, p0, p1), derivative(x, p0, p1)) as torch expressions
_REF: Dict[str, Tuple[Callable, Callable]] = {
    "exp": (lambda x, a, b: torch.exp(x), lambda x, a, b: torch.exp(x)),
    "log": (lambda x, a, b: torch.log(x), lambda x, a, b: 1 / x),
    "sqrt": (lambda x, a, b: torch.sqrt(x), lambda x, a, b: 0.5 / torch.sqrt(x)),
    "sin": (lambda x, a, b: torch.sin(x), lambda x, a, b: torch.cos(x)),
    "cos": (lambda x, a, b: torch.cos(x), lambda x, a, b: -torch.sin(x)),
    "tan": (lambda x, a, b: torch.tan(x), lambda x, a, b: 1 / torch.cos(x) ** 2),
    "abs": (lambda x, a, b: torch.abs(x), lambda x, a, b: torch.sign(x)),
    "reciprocal": (lambda x, a, b: 1 / x, lambda x, a, b: -1 / (x * x)),
    "square": (lambda x, a, b: x * x, lambda x, a, b: 2 * x),
    "relu": (lambda x, a, b: torch.relu(x), lambda x, a, b: (x > 0).to(x.dtype)),
    "selu": (lambda x, a, b: torch.where(x > 0, _SELU_S * x, _SELU_S * _SELU_A * (torch.exp(x) - 1)),
             lambda x, a, b: torch.where(x > 0, torch.full_like(x, _SELU_S), _SELU_S * _SELU_A * torch.exp(x))),
    "sigmoid": (lambda x, a, b: torch.sigmoid(x), lambda x, a, b: torch.sigmoid(x) * (1 - torch.sigmoid(x))),
    "tanh": (lambda x, a, b: torch.tanh(x), lambda x, a, b: 1 - torch.tanh(x) ** 2),
    "hardtanh": (lambda x, a, b: torch.clamp(x, -1, 1), lambda x, a, b: ((x > -1) & (x < 1)).to(x.dtype)),
    "hardsigmoid": (lambda x, a, b: torch.clamp(x / 6 + 0.5, 0, 1),
                    lambda x, a, b: ((x > -3) & (x < 3)).to(x.dtype) / 6),
    "softplus": (lambda x, a, b: _sp(x), lambda x, a, b: torch.where(x > 20, torch.ones_like(x), torch.sigmoid(x))),
    "softsign": (lambda x, a, b: x / (1 + torch.abs(x)), lambda x, a, b: 1 / (1 + torch.abs(x)) ** 2),
    "gelu": (lambda x, a, b: 0.5 * x * (1 + torch.tanh(_K0 * (x + _K1 * x ** 3))),
             lambda x, a, b: _dgelu_tanh(x)),
    "geluexact": (lambda x, a, b: 0.5 * x * (1 + torch.erf(x / math.sqrt(2))),
                  lambda x, a, b: 0.5 * (1 + torch.erf(x / math.sqrt(2))) + x * torch.exp(-0.5 * x * x) / math.sqrt(2 * math.pi)),
    "silu": (lambda x, a, b: x * torch.sigmoid(x),
             lambda x, a, b: torch.sigmoid(x) * (1 + x * (1 - torch.sigmoid(x)))),
    "hardswish": (lambda x, a, b: x * torch.clamp(x + 3, 0, 6) / 6,
                  lambda x, a, b: torch.where(x < -3, torch.zeros_like(x), torch.where(x > 3, torch.ones_like(x), (2 * x + 3) / 6))),
    "mish": (lambda x, a, b: x * torch.tanh(_sp(x)),
             lambda x, a, b: torch.tanh(_sp(x)) + x * (1 - torch.tanh(_sp(x)) ** 2) * torch.sigmoid(x)),
    "relu6": (lambda x, a, b: torch.clamp(x, 0, 6), lambda x, a, b: ((x > 0) & (x < 6)).to(x.dtype)),
    "logsigmoid": (lambda x, a, b: -_sp(-x), lambda x, a, b: torch.sigmoid(-x)),
    "tanhshrink": (lambda x, a, b: x - torch.tanh(x), lambda x, a, b: torch.tanh(x) ** 2),
    "pow": (lambda x, a, b: torch.pow(x, a), lambda x, a, b: a * torch.pow(x, a - 1)),
    "clip": (lambda x, a, b: torch.clamp(x, a, b), lambda x, a, b: ((x >= a) & (x <= b)).to(x.dtype)),
    "leakyrelu": (lambda x, a, b: torch.where(x > 0, x, a * x),
                  lambda x, a, b: torch.where(x > 0, torch.ones_like(x), torch.full_like(x, a))),
    "elu": (lambda x, a, b: torch.where(x > 0, x, a * (torch.exp(x) - 1)),
            lambda x, a, b: torch.where(x > 0, torch.ones_like(x), a * torch.exp(x))),
    "hardshrink": (lambda x, a, b: torch.where(torch.abs(x) > a, x, torch.zeros_like(x)),
                   lambda x, a, b: (torch.abs(x) > a).to(x.dtype)),
    "softshrink": (lambda x, a, b: torch.where(x > a, x - a, torch.where(x < -a, x + a, torch.zeros_like(x))),
                   lambda x, a, b: (torch.abs(x) > a).to(x.dtype)),
    "softplusbeta": (lambda x, a, b: torch.where(a * x > b, x, torch.log1p(torch.exp(torch.clamp(a * x, max=b))) / a),
                     lambda x, a, b: torch.where(a * x > b, torch.ones_like(x), torch.sigmoid(a * x))),
    "threshold": (lambda x, a, b: torch.where(x > a, x, torch.full_like(x, b)), lambda x, a, b: (x > a).to(x.dtype)),
    "celu": (lambda x, a, b: torch.clamp(x, min=0) + torch.clamp(a * (torch.exp(x / a) - 1), max=0),
             lambda x, a, b: torch.where(x > 0, torch.ones_like(x), torch.exp(x / a))),
    "neg": (lambda x, a, b: -x, lambda x, a, b: -torch.ones_like(x)),
    "scale_add": (lambda x, a, b: a * x + b, lambda x, a, b: torch.full_like(x, a)),
}


def _dgelu_tanh(x):
    t = torch.tanh(_K0 * (x + _K1 * x ** 3))
    return 0.5 * (1 + t) + 0.5 * x * (1 - t * t) * _K0 * (1 + 3 * _K1 * x * x)


_NATIVE_DT = (torch.bfloat16, torch.float16, torch.float32, torch.float64)


def _native(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype in _NATIVE_DT


def unary_forward(name: str, x: torch.Tensor, p0: float = 0.0, p1: float = 0.0) -> torch.Tensor:
    if name not in UNARY_IDS:
        raise KeyError(f"unknown unary op {name!r}")
    if not _native(x):
        if x.is_cuda:
            raise TypeError(f"unary {name}: no CUDA kernel for dtype {x.dtype}")
        ct = x.dtype if x.dtype in (torch.float32, torch.float64) else torch.float32
        return _REF[name][0](x.to(ct), p0, p1).to(x.dtype)
    xc = x.contiguous()
    y = torch.empty_like(xc)
    _l.call("gb_unary_fwd", _l.I(UNARY_IDS[name]), _l.I(_l.dtype_code(x.dtype)), _l.ptr(xc), _l.ptr(y),
            _l.L(xc.numel()), _l.D(p0), _l.D(p1), _l.stream_ptr())
    return y


def unary_backward(name: str, x: torch.Tensor, dy: torch.Tensor, p0: float = 0.0, p1: float = 0.0) -> torch.Tensor:
    """dx = dy * f'(x)."""
    if not _native(x):
        if x.is_cuda:
            raise TypeError(f"unary {name}: no CUDA kernel for dtype {x.dtype}")
        ct = x.dtype if x.dtype in (torch.float32, torch.float64) else torch.float32
        return (dy.to(ct) * _REF[name][1](x.to(ct), p0, p1)).to(x.dtype)
    xc, dyc = x.contiguous(), dy.contiguous()
    dx = torch.empty_like(xc)
    _l.call("gb_unary_bwd", _l.I(UNARY_IDS[name]), _l.I(_l.dtype_code(x.dtype)), _l.ptr(xc), _l.ptr(dyc),
            _l.ptr(dx), _l.L(xc.numel()), _l.D(p0), _l.D(p1), _l.stream_ptr())
    return dx


class _Unary(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, name, p0, p1):
        ctx.save_for_backward(x)
        ctx.meta = (name, p0, p1)
        return unary_forward(name, x, p0, p1)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        name, p0, p1 = ctx.meta
        return unary_backward(name, x, dy, p0, p1), None, None, None


def unary(name: str, x: torch.Tensor, p0: float = 0.0, p1: float = 0.0) -> torch.Tensor:
    """Differentiable unary op by name (kernel forward, kernel backward)."""
    if not (x.requires_grad and torch.is_grad_enabled()):
        return unary_forward(name, x, float(p0), float(p1))      # nothing to record: skip the tape node
    return _Unary.apply(x, name, float(p0), float(p1))


def _bcast_strides(t: torch.Tensor, shape) -> list:
    """Element strides of ``t`` seen through ``shape`` (0 where broadcast)."""
    nd = len(shape)
    ts = [1] * (nd - t.dim()) + list(t.shape)
    st = [0] * (nd - t.dim()) + list(t.stride())
    return [0 if ts[i] == 1 and shape[i] != 1 else st[i] for i in range(nd)]


def binary_forward(name: str, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    if a.dtype != b.dtype:
        dt = torch.promote_types(a.dtype, b.dtype)
        a, b = a.to(dt), b.to(dt)
    if not _native(a):
        if a.is_cuda:
            raise TypeError(f"binary {name}: no CUDA kernel for dtype {a.dtype}")
        return {"add": torch.add, "sub": torch.sub, "mul": torch.mul, "div": torch.div}[name](a, b)
    if a.shape == b.shape and a.is_contiguous() and b.is_contiguous():
        # the common case, tested before any shape arithmetic (broadcast_shapes alone costs more
        # host time than the rest of this function)
        out = torch.empty(a.shape, dtype=a.dtype, device=a.device)
        _l.call("gb_binary", _l.I(BINARY_IDS[name]), _l.I(_l.dtype_code(a.dtype)), _l.ptr(a), _l.ptr(b),
                _l.ptr(out), _l.L(out.numel()), _l.I(0), None, None, None, _l.stream_ptr())
        return out
    shape = torch.broadcast_shapes(a.shape, b.shape)
    out = torch.empty(shape, dtype=a.dtype, device=a.device)
    n = out.numel()
    if len(shape) > 6:
        a, b = a.expand(shape).contiguous(), b.expand(shape).contiguous()
        return binary_forward(name, a, b)
    sa, sb = _bcast_strides(a, shape), _bcast_strides(b, shape)
    nd = max(len(shape), 1)
    shp = list(shape) if len(shape) else [1]
    arr = _l.L * nd
    _l.call("gb_binary", _l.I(BINARY_IDS[name]), _l.I(_l.dtype_code(a.dtype)), _l.ptr(a), _l.ptr(b),
            _l.ptr(out), _l.L(n), _l.I(nd), arr(*shp), arr(*(sa or [0])), arr(*(sb or [0])),
            _l.stream_ptr())
    return out


def sum_to_shape(g: torch.Tensor, shape) -> torch.Tensor:
    """Un-broadcast: sums ``g`` down to ``shape`` (reference: tensor/broadcast.go:92-118)."""
    from .reduce import reduce_axis
    if tuple(g.shape) == tuple(shape):
        return g
    lead = g.dim() - len(shape)
    for _ in range(lead):
        g = reduce_axis(g, 0, "sum", keepdim=False)
    for i, s in enumerate(shape):
        if s == 1 and g.shape[i] != 1:
            g = reduce_axis(g, i, "sum", keepdim=True)
    return g


class _Binary(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, name):
        ctx.name = name
        ctx.save_for_backward(a, b)
        return binary_forward(name, a, b)

    @staticmethod
    def backward(ctx, g):
        a, b = ctx.saved_tensors
        name = ctx.name
        ga = gb = None
        if name == "add":
            ga, gb = g, g
        elif name == "sub":
            ga, gb = g, unary_forward("neg", g)
        elif name == "mul":
            ga, gb = binary_forward("mul", g, b), binary_forward("mul", g, a)
        else:
            ga = binary_forward("div", g, b)
            gb = unary_forward("neg", binary_forward("div", binary_forward("mul", g, a), binary_forward("mul", b, b)))
        if ctx.needs_input_grad[0]:
            ga = sum_to_shape(ga, a.shape).to(a.dtype)
        else:
            ga = None
        if ctx.needs_input_grad[1]:
            gb = sum_to_shape(gb, b.shape).to(b.dtype)
        else:
            gb = None
        return ga, gb, None


def binary(name: str, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Differentiable broadcasting add / sub / mul / div."""
    if name not in BINARY_IDS:
        raise KeyError(f"unknown binary op {name!r}")
    if not ((a.requires_grad or b.requires_grad) and torch.is_grad_enabled()):
        return binary_forward(name, a, b)
    return _Binary.apply(a, b, name)


def cast(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """dtype conversion with round-to-nearest-even (not differentiable by itself)."""
    if x.dtype == dtype:
        return x
    if not (_native(x) and dtype in _NATIVE_DT):
        return x.to(dtype)
    xc = x.contiguous()
    y = torch.empty(xc.shape, dtype=dtype, device=x.device)
    _l.call("gb_cast", _l.I(_l.dtype_code(x.dtype)), _l.I(_l.dtype_code(dtype)), _l.ptr(xc), _l.ptr(y),
            _l.L(xc.numel()), _l.stream_ptr())
    return y

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence

import torch

from ..ops import elementwise as _ew
from ..ops.linear import matmul as _matmul
from ..ops.reduce import reduce_axis as _reduce
from ..ops.softmax import log_softmax as _log_softmax, softmax as _softmax

Tensor = torch.Tensor
Float64, Float32, Float16, BFloat16 = torch.float64, torch.float32, torch.float16, torch.bfloat16

__all__: List[str] = []


def _export(fn):
    __all__.append(fn.__name__)
    return fn


def op_error(op: str, msg: str):
    """Uniform error text ``tensor.<Op>: ...`` (tensor/internal.go:10-20)."""
    return ValueError(f"tensor.{op}: {msg}")


# ---------------------------------------------------------------------------------------
# constructors (tensor/tensor.go:33-178)
# ---------------------------------------------------------------------------------------
@_export
def New(data, *shape, dtype=torch.float64, device=None, requires_grad=False) -> Tensor:
    t = torch.as_tensor(data, dtype=dtype, device=device)
    if shape:
        n = 1
        for s in shape:
            n *= s
        if n != t.numel():
            raise op_error("New", f"data has {t.numel()} elements, shape {shape} needs {n}")
        t = t.reshape(*shape)
    t = t.clone()
    return t.requires_grad_(requires_grad)


@_export
def NewLike(t: Tensor, data) -> Tensor:
    return torch.as_tensor(data, dtype=t.dtype, device=t.device).reshape(t.shape).clone()


@_export
def NewTyped(data, dtype, *shape, device=None) -> Tensor:
    return New(data, *shape, dtype=dtype, device=device)


@_export
def Zeros(*shape, dtype=torch.float64, device=None) -> Tensor:
    return torch.zeros(*shape, dtype=dtype, device=device)


@_export
def Ones(*shape, dtype=torch.float64, device=None) -> Tensor:
    return torch.ones(*shape, dtype=dtype, device=device)


@_export
def Full(value: float, *shape, dtype=torch.float64, device=None) -> Tensor:
    return torch.full(shape, value, dtype=dtype, device=device)


@_export
def Randn(*shape, dtype=torch.float64, device=None) -> Tensor:
    return torch.randn(*shape, dtype=torch.float64).to(dtype=dtype, device=device)


@_export
def Uniform(lo: float, hi: float, *shape, dtype=torch.float64, device=None) -> Tensor:
    return torch.empty(*shape, dtype=torch.float64).uniform_(lo, hi).to(dtype=dtype, device=device)


@_export
def Arange(start: float, stop: float, step: float = 1.0, dtype=torch.float64, device=None) -> Tensor:
    return torch.arange(start, stop, step, dtype=dtype, device=device)


@_export
def Eye(n: int, dtype=torch.float64, device=None) -> Tensor:
    return torch.eye(n, dtype=dtype, device=device)


@_export
def Scalar(v: float, dtype=torch.float64, device=None) -> Tensor:
    """A 0-d tensor."""
    return torch.tensor(v, dtype=dtype, device=device)


@_export
def Copy(t: Tensor) -> Tensor:
    return t.detach().clone()


@_export
def Numel(t: Tensor) -> int:
    return t.numel()


@_export
def Item(t: Tensor) -> float:
    if t.numel() != 1:
        raise op_error("Item", f"tensor has {t.numel()} elements")
    return float(t.item())


@_export
def SetRequiresGrad(t: Tensor, flag: bool = True) -> Tensor:
    return t.requires_grad_(flag)


@_export
def ZeroGrad(t: Tensor) -> None:
    t.grad = None


@_export
def Backward(t: Tensor) -> None:
    """Scalar-only backward, seeding the gradient with 1 (tensor/autograd.go:52-99)."""
    if t.numel() != 1:
        raise op_error("Backward", "only scalar tensors can start a backward pass")
    t.backward()


@_export
def MakeNode(out_fn: Callable[..., Tensor], name: str, inputs: Sequence[Tensor],
             backward: Callable[[Tensor], Sequence[Optional[Tensor]]]) -> Tensor:
    """Custom-op escape hatch (tensor/autograd.go:153-178): evaluates ``out_fn(*inputs)``
    without a tape and attaches ``backward(grad_out) -> grads of inputs``."""

    class _Node(torch.autograd.Function):
        @staticmethod
        def forward(ctx, *xs):
            return out_fn(*xs)

        @staticmethod
        def backward(ctx, g):
            gs = backward(g)
            return tuple(gs)

    _Node.__name__ = name
    return _Node.apply(*inputs)


# ---------------------------------------------------------------------------------------
# unary-op registry (tensor/registry.go:20-110)
# ---------------------------------------------------------------------------------------
@dataclass
class UnaryOpDef:
    Name: str
    Fwd: Callable[[Tensor], Tensor]
    Bwd: Callable[[Tensor, Tensor], Tensor]  # (x, grad_out) -> grad_in
    Kind: int = -1                            # native kernel id, -1 = host expression only


_REGISTRY: Dict[str, UnaryOpDef] = {}


@_export
def RegisterUnary(d: UnaryOpDef) -> None:
    if not d.Name:
        raise op_error("RegisterUnary", "empty name")
    if d.Name in _REGISTRY:
        raise op_error("RegisterUnary", f"duplicate op {d.Name!r}")
    if d.Fwd is None or d.Bwd is None:
        raise op_error("RegisterUnary", f"op {d.Name!r} needs both Fwd and Bwd")
    _REGISTRY[d.Name] = d


@_export
def LookupUnary(name: str) -> Optional[UnaryOpDef]:
    return _REGISTRY.get(name)


@_export
def UnaryOpNames() -> List[str]:
    return sorted(_REGISTRY)


def _builtin(name: str) -> UnaryOpDef:
    return UnaryOpDef(name, lambda x, n=name: _ew.unary_forward(n, x),
                      lambda x, g, n=name: _ew.unary_backward(n, x, g), _ew.UNARY_IDS[name])


for _n in _ew.REGISTERED_UNARY:
    RegisterUnary(_builtin(_n))


class _UserUnary(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, d):
        ctx.save_for_backward(x)
        ctx.d = d
        return d.Fwd(x)

    @staticmethod
    def backward(ctx, g):
        (x,) = ctx.saved_tensors
        return ctx.d.Bwd(x, g), None


@_export
def Unary(x: Tensor, name: str) -> Tensor:
    """Applies a registered op by name, with autograd."""
    d = _REGISTRY.get(name)
    if d is None:
        raise op_error("Unary", f"unknown op {name!r}")
    if d.Kind >= 0:
        return _ew.unary(name, x)
    return _UserUnary.apply(x, d)


def _mk_unary(go_name: str, reg_name: str):
    def f(x: Tensor) -> Tensor:
        return _ew.unary(reg_name, x)
    f.__name__ = go_name
    f.__doc__ = f"Elementwise ``{reg_name}`` (kernel forward and backward)."
    return _export(f)


Exp = _mk_unary("Exp", "exp"); Log = _mk_unary("Log", "log"); Sqrt = _mk_unary("Sqrt", "sqrt")
Sin = _mk_unary("Sin", "sin"); Cos = _mk_unary("Cos", "cos"); Tan = _mk_unary("Tan", "tan")
Abs = _mk_unary("Abs", "abs"); Reciprocal = _mk_unary("Reciprocal", "reciprocal")
Square = _mk_unary("Square", "square"); ReLU = _mk_unary("ReLU", "relu"); SELU = _mk_unary("SELU", "selu")
Sigmoid = _mk_unary("Sigmoid", "sigmoid"); Tanh = _mk_unary("Tanh", "tanh")
HardTanh = _mk_unary("HardTanh", "hardtanh"); HardSigmoid = _mk_unary("HardSigmoid", "hardsigmoid")
Softplus = _mk_unary("Softplus", "softplus"); Softsign = _mk_unary("Softsign", "softsign")
GELU = _mk_unary("GELU", "gelu"); GELUExact = _mk_unary("GELUExact", "geluexact")
SiLU = _mk_unary("SiLU", "silu"); Swish = _mk_unary("Swish", "silu"); HardSwish = _mk_unary("HardSwish", "hardswish")
Mish = _mk_unary("Mish", "mish"); ReLU6 = _mk_unary("ReLU6", "relu6")
LogSigmoid = _mk_unary("LogSigmoid", "logsigmoid"); Tanhshrink = _mk_unary("Tanhshrink", "tanhshrink")
Neg = _mk_unary("Neg", "neg")


@_export
def Pow(x, p: float): return _ew.unary("pow", x, p)
@_export
def Clip(x, lo: float, hi: float): return _ew.unary("clip", x, lo, hi)
@_export
def LeakyReLU(x, alpha: float = 0.01): return _ew.unary("leakyrelu", x, alpha)
@_export
def ELU(x, alpha: float = 1.0): return _ew.unary("elu", x, alpha)
@_export
def CELU(x, alpha: float = 1.0): return _ew.unary("celu", x, alpha)
@_export
def Hardshrink(x, lambd: float = 0.5): return _ew.unary("hardshrink", x, lambd)
@_export
def Softshrink(x, lambd: float = 0.5): return _ew.unary("softshrink", x, lambd)
@_export
def SoftplusBeta(x, beta: float = 1.0, threshold: float = 20.0): return _ew.unary("softplusbeta", x, beta, threshold)
@_export
def Threshold(x, th: float, value: float): return _ew.unary("threshold", x, th, value)
@_export
def RReLU(x, lower: float = 1 / 8, upper: float = 1 / 3): return _ew.unary("leakyrelu", x, (lower + upper) / 2)


# ---------------------------------------------------------------------------------------
# binary ops with NumPy broadcasting (tensor/ops_binary.go, tensor/broadcast.go)
# ---------------------------------------------------------------------------------------
def _t(x, like: Tensor) -> Tensor:
    return x if isinstance(x, torch.Tensor) else torch.tensor(x, dtype=like.dtype, device=like.device)


@_export
def Add(a, b): return _ew.binary("add", a, _t(b, a))
@_export
def Sub(a, b): return _ew.binary("sub", a, _t(b, a))
@_export
def Mul(a, b): return _ew.binary("mul", a, _t(b, a))
@_export
def Div(a, b): return _ew.binary("div", a, _t(b, a))
@_export
def AddScalar(a, s: float): return _ew.unary("scale_add", a, 1.0, s)
@_export
def SubScalar(a, s: float): return _ew.unary("scale_add", a, 1.0, -s)
@_export
def MulScalar(a, s: float): return _ew.unary("scale_add", a, s, 0.0)
@_export
def DivScalar(a, s: float): return _ew.unary("scale_add", a, 1.0 / s, 0.0)


@_export
def BroadcastShapes(a: Sequence[int], b: Sequence[int]):
    try:
        return tuple(torch.broadcast_shapes(tuple(a), tuple(b)))
    except RuntimeError:
        raise op_error("broadcast", f"shapes {tuple(a)} and {tuple(b)} are not broadcastable") from None


# ---------------------------------------------------------------------------------------
# matmul (tensor/ops_matmul.go:17-105)
# ---------------------------------------------------------------------------------------
@_export
def MatMul(a: Tensor, b: Tensor) -> Tensor:
    """2-D fast path; rank >= 3 is batched with NumPy batch-dimension broadcasting."""
    if a.dim() < 1 or b.dim() < 1:
        raise op_error("MatMul", "operands must have rank >= 1")
    return _matmul(a, b)


@_export
def BMM(a: Tensor, b: Tensor) -> Tensor:
    """Strict batched product: (B,m,k) x (B,k,n)."""
    if a.dim() != 3 or b.dim() != 3 or a.shape[0] != b.shape[0] or a.shape[2] != b.shape[1]:
        raise op_error("BMM", f"expected (B,m,k) x (B,k,n), got {tuple(a.shape)} x {tuple(b.shape)}")
    return _matmul(a, b)


# ---------------------------------------------------------------------------------------
# reductions (tensor/ops_reduce.go:6-271)
# ---------------------------------------------------------------------------------------
class _ReduceAxis(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, axis, op, keepdim):
        axis = axis % x.dim()
        y = _reduce(x, axis, op, keepdim)
        ctx.meta = (axis, op, keepdim, x.shape)
        if op in ("max", "min"):
            idx = _reduce(x, axis, "arg" + op, True)
            ctx.save_for_backward(idx)
        return y

    @staticmethod
    def backward(ctx, g):
        axis, op, keepdim, shape = ctx.meta
        if not keepdim:
            g = g.unsqueeze(axis)
        if op == "sum":
            return g.expand(shape), None, None, None
        if op == "mean":
            return (g / shape[axis]).expand(shape), None, None, None
        (idx,) = ctx.saved_tensors
        out = torch.zeros(shape, dtype=g.dtype, device=g.device)
        out.scatter_(axis, idx, g)  # the first extremum receives the gradient
        return out, None, None, None


def _axis(op, x, axis):
    if not -x.dim() <= axis < x.dim():
        raise op_error(op, f"axis {axis} out of range for rank {x.dim()}")
    return axis % x.dim()


@_export
def SumAxis(x, axis: int, keepdim: bool = False): return _ReduceAxis.apply(x, _axis("SumAxis", x, axis), "sum", keepdim)
@_export
def MeanAxis(x, axis: int, keepdim: bool = False): return _ReduceAxis.apply(x, _axis("MeanAxis", x, axis), "mean", keepdim)
@_export
def MaxAxis(x, axis: int, keepdim: bool = False): return _ReduceAxis.apply(x, _axis("MaxAxis", x, axis), "max", keepdim)
@_export
def MinAxis(x, axis: int, keepdim: bool = False): return _ReduceAxis.apply(x, _axis("MinAxis", x, axis), "min", keepdim)
@_export
def Sum(x): return _ReduceAxis.apply(x.reshape(-1), 0, "sum", False)
@_export
def Mean(x): return _ReduceAxis.apply(x.reshape(-1), 0, "mean", False)
@_export
def Max(x): return _ReduceAxis.apply(x.reshape(-1), 0, "max", False)
@_export
def Min(x): return _ReduceAxis.apply(x.reshape(-1), 0, "min", False)
@_export
def ArgMax(x, axis: int): return _reduce(x.detach(), _axis("ArgMax", x, axis), "argmax")
@_export
def ArgMin(x, axis: int): return _reduce(x.detach(), _axis("ArgMin", x, axis), "argmin")
@_export
def Softmax(x, axis: int = -1): return _softmax(x, axis)
@_export
def LogSoftmax(x, axis: int = -1): return _log_softmax(x, axis)


# ---------------------------------------------------------------------------------------
# shape ops (tensor/ops_shape.go:5-241): views where the layout allows, no hidden copies
# ---------------------------------------------------------------------------------------
@_export
def Reshape(x, *shape): return x.reshape(*shape)
View = Reshape; __all__.append("View")
@_export
def Flatten(x): return x.reshape(-1)
@_export
def Transpose(x):
    if x.dim() < 2:
        raise op_error("Transpose", "needs rank >= 2")
    return x.transpose(-1, -2)
T = Transpose; __all__.append("T")
@_export
def Permute(x, *dims): return x.permute(*dims)
@_export
def Squeeze(x, axis: Optional[int] = None): return x.squeeze() if axis is None else x.squeeze(axis)
@_export
def Unsqueeze(x, axis: int): return x.unsqueeze(axis)
@_export
def Expand(x, *shape): return x.expand(*shape)
@_export
def Concat(ts: Sequence[Tensor], axis: int = 0): return torch.cat(list(ts), dim=axis)
@_export
def Stack(ts: Sequence[Tensor], axis: int = 0): return torch.stack(list(ts), dim=axis)


# ---------------------------------------------------------------------------------------
# extra ops (tensor/ops_extra.go:59-368) and index ops (tensor/ops_index.go:7-125)
# ---------------------------------------------------------------------------------------
@_export
def Tril(x, k: int = 0): return torch.tril(x, k)
@_export
def Triu(x, k: int = 0): return torch.triu(x, k)
@_export
def Where(cond, a, b): return torch.where(cond.bool() if cond.dtype != torch.bool else cond, a, _t(b, a))
@_export
def MaskedFill(x, mask, value: float): return x.masked_fill(mask.bool(), value)
@_export
def Cumsum(x, axis: int):
    """Inclusive prefix sum along ``axis`` (scan kernel on CUDA tensors)."""
    from ..ops.shape import cumsum as _cumsum
    return _cumsum(x, axis)
@_export
def Flip(x, *axes): return torch.flip(x, dims=list(axes))
@_export
def Repeat(x, *reps): return x.repeat(*reps)
Tile = Repeat; __all__.append("Tile")
@_export
def Split(x, size: int, axis: int = 0): return list(torch.split(x, size, dim=axis))
@_export
def Chunk(x, n: int, axis: int = 0): return list(torch.chunk(x, n, dim=axis))


@_export
def Gather(x, axis: int, index):
    """out[i][j] = x[i][index[i][j]] along ``axis``; scatter-add backward."""
    return torch.gather(x, axis, index.long())


@_export
def IndexSelect(x, axis: int, index):
    """Rows of ``x`` along ``axis``; axis 0 of a matrix uses the embedding kernels."""
    idx = index.long().reshape(-1)
    if axis % x.dim() == 0 and x.dim() == 2:
        from ..ops.embedding import embedding
        return embedding(x, idx)
    return torch.index_select(x, axis, idx)


@_export
def ArgWhere(x): return torch.nonzero(x)


# ---------------------------------------------------------------------------------------
# dtype (tensor/dtype.go:17-186)
# ---------------------------------------------------------------------------------------
class _AsType(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dtype):
        ctx.src = x.dtype
        return _ew.cast(x, dtype)

    @staticmethod
    def backward(ctx, g):
        return _ew.cast(g, ctx.src), None  # straight-through


@_export
def AsType(x, dtype): return _AsType.apply(x, dtype)
To = AsType; __all__.append("To")


@_export
def RoundTo(x, dtype):
    """The reference's precision emulation: round values to ``dtype`` (nearest-even) but keep
    the storage dtype (tensor/dtype.go:50-70)."""
    return _ew.cast(_ew.cast(x, dtype), x.dtype)


@_export
def Promote(a, b): return torch.promote_types(a, b)


# ---------------------------------------------------------------------------------------
# dispatch policy (tensor/dispatch.go:44-113)
# ---------------------------------------------------------------------------------------
@dataclass
class DispatchPolicy:
    """Element-count thresholds above which the reference sent an op to its accelerator
    backend.  Here placement follows the tensor's device, so the policy is informational:
    it is stored and returned for code that reads it."""
    UnaryMinElems: int = 1 << 16
    BinaryMinElems: int = (1 << 63) - 1


_policy = DispatchPolicy()


@_export
def SetDispatchPolicy(p: DispatchPolicy) -> DispatchPolicy:
    global _policy
    old, _policy = _policy, p
    return old


@_export
def GetDispatchPolicy() -> DispatchPolicy:
    return _policy


# ---------------------------------------------------------------------------------------
# names of the reference's types
# ---------------------------------------------------------------------------------------
DType = torch.dtype                         # tensor/dtype.go:17 (an enum there, real dtypes here)
from ..backend import UnaryKind             # noqa: E402  (tensor/dispatch.go:29 re-exports it too)

UnaryNone, UnaryReLU, UnarySigmoid, UnaryTanh = (UnaryKind.NoneKind, UnaryKind.ReLU, UnaryKind.Sigmoid,
                                                 UnaryKind.Tanh)
UnaryExp, UnaryLog, UnaryGELU, UnarySiLU, UnaryGELUExact = (UnaryKind.Exp, UnaryKind.Log, UnaryKind.GELU,
                                                            UnaryKind.SiLU, UnaryKind.GELUExact)


@_export
def DTypeString(dt: torch.dtype) -> str:
    """PyTorch-style name of a dtype: ``"float32"`` (tensor/dtype.go:28-37)."""
    return str(dt).replace("torch.", "")


@_export
def String(t: Tensor) -> str:
    """The reference's print format (tensor/tensor.go:152-170): shape, up to 16 values (the
    first and last 8 beyond that), the dtype unless float64, and the gradient flag."""
    flat = t.detach().reshape(-1)
    vals = lambda v: "[" + " ".join(f"{x:g}" for x in v.to("cpu", torch.float64).tolist()) + "]"
    body = vals(flat) if flat.numel() <= 16 else f"[{vals(flat[:8])} ... {vals(flat[-8:])}]"
    out = f"Tensor(shape=[{' '.join(str(d) for d in t.shape)}], data={body}"
    if t.dtype != torch.float64:
        out += ", dtype=" + DTypeString(t.dtype)
    if t.requires_grad:
        out += ", requires_grad=true"
    return out + ")"


@dataclass
class Function:
    """A tape node described by value (tensor/autograd.go:36-41): ``Backward(grad, saved,
    inputs)`` returns one gradient (or None) per input.  ``Apply(out_fn)`` evaluates
    ``out_fn(*Inputs)`` off the tape and records the node, which is what ``MakeNode`` does
    with a closure."""
    Name: str
    Inputs: Sequence[Tensor]
    Saved: Sequence[object] = ()
    Backward: Optional[Callable[[Tensor, Sequence[object], Sequence[Tensor]], Sequence[Optional[Tensor]]]] = None

    def Apply(self, out_fn: Callable[..., Tensor]) -> Tensor:
        if self.Backward is None:
            raise op_error("Function.Apply", f"node {self.Name!r} has no Backward")
        return MakeNode(out_fn, self.Name, self.Inputs,
                        lambda g: self.Backward(g, self.Saved, self.Inputs))


__all__ += ["Tensor", "Float64", "Float32", "Float16", "BFloat16", "UnaryOpDef", "DispatchPolicy", "op_error", "DType", "UnaryKind", "Function",
            "UnaryNone", "UnaryReLU", "UnarySigmoid", "UnaryTanh", "UnaryExp", "UnaryLog", "UnaryGELU",
            "UnarySiLU", "UnaryGELUExact"]

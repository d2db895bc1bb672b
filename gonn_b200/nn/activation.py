"""Activation modules (nn/activation.go:21-332).  Fixed kinds route through the
unary-op registry by name; parameterised kinds pass their constants."""
from __future__ import annotations

import torch

from ..ops import elementwise as _ew
from ..ops.softmax import log_softmax as _log_softmax, softmax as _softmax
from .module import Module


class Activation(Module):
    """Generic activation: ``kind`` is a registry name; ``alpha`` / ``beta`` are the
    op's parameters (e.g. LeakyReLU slope, ELU alpha, Softplus beta/threshold)."""

    def __init__(self, kind: str, alpha: float = 0.0, beta: float = 0.0):
        super().__init__()
        # built-in kinds are op ids of the elementwise kernel; any other name must be in the
        # tensor package's registry (RegisterUnary), as in the reference (nn/activation.go)
        self._user = kind not in _ew.UNARY_IDS
        if self._user:
            from ..tensor import api as _api
            if _api.LookupUnary(kind) is None:
                raise KeyError(f"nn.Activation: unknown kind {kind!r}")
        self.kind, self.alpha, self.beta = kind, float(alpha), float(beta)

    def forward(self, x):
        if self._user:
            from ..tensor import api as _api
            return _api.Unary(x, self.kind)
        return _ew.unary(self.kind, x, self.alpha, self.beta)

    def extra_repr(self):
        return self.kind


def ReLU(): return Activation("relu")
def ReLU6(): return Activation("relu6")
def Sigmoid(): return Activation("sigmoid")
def Tanh(): return Activation("tanh")
def GELU(): return Activation("gelu")          # tanh approximation, the reference's default
def GELUApprox(): return Activation("gelu")
def GELUExact(): return Activation("geluexact")
def SiLU(): return Activation("silu")
def Swish(): return Activation("silu")
def SELU(): return Activation("selu")
def HardTanh(): return Activation("hardtanh")
def HardSigmoid(): return Activation("hardsigmoid")
def HardSwish(): return Activation("hardswish")
def Mish(): return Activation("mish")
def Softplus(): return Activation("softplus")
def Softsign(): return Activation("softsign")
def LogSigmoid(): return Activation("logsigmoid")
def Tanhshrink(): return Activation("tanhshrink")
def LeakyReLU(negative_slope: float = 0.01): return Activation("leakyrelu", negative_slope)
def ELU(alpha: float = 1.0): return Activation("elu", alpha)
def CELU(alpha: float = 1.0): return Activation("celu", alpha)
def Hardshrink(lambd: float = 0.5): return Activation("hardshrink", lambd)
def Softshrink(lambd: float = 0.5): return Activation("softshrink", lambd)
def Threshold(threshold: float, value: float): return Activation("threshold", threshold, value)
def SoftplusWith(beta: float = 1.0, threshold: float = 20.0): return Activation("softplusbeta", beta, threshold)


_BY_NAME = {"relu": ReLU, "relu6": ReLU6, "sigmoid": Sigmoid, "tanh": Tanh, "gelu": GELU,
            "geluexact": GELUExact, "silu": SiLU, "swish": SiLU, "selu": SELU, "hardtanh": HardTanh,
            "hardsigmoid": HardSigmoid, "hardswish": HardSwish, "mish": Mish, "softplus": Softplus,
            "softsign": Softsign, "logsigmoid": LogSigmoid, "tanhshrink": Tanhshrink,
            "leakyrelu": LeakyReLU, "elu": ELU, "celu": CELU}


def ActivationByName(name: str) -> Activation:
    try:
        return _BY_NAME[name.lower()]()
    except KeyError:
        raise KeyError(f"nn.ActivationByName: unknown activation {name!r}") from None


class Softmax(Module):
    def __init__(self, dim: int = -1):
        super().__init__()
        self.dim = dim

    def forward(self, x):
        return _softmax(x, self.dim)


class LogSoftmax(Module):
    def __init__(self, dim: int = -1):
        super().__init__()
        self.dim = dim

    def forward(self, x):
        return _log_softmax(x, self.dim)


class Softmin(Module):
    def __init__(self, dim: int = -1):
        super().__init__()
        self.dim = dim

    def forward(self, x):
        return _softmax(_ew.unary("neg", x), self.dim)


class Softmax2d(Module):
    """Softmax over the channel dim of (N, C, H, W) or (C, H, W)."""

    def forward(self, x):
        return _softmax(x, -3)


class PReLU(Module):
    """max(0,x) + a*min(0,x) with learnable slope(s), initial 0.25 (nn/activation.go:237)."""

    def __init__(self, num_parameters: int = 1, init: float = 0.25, *, dtype=torch.float32, device=None):
        super().__init__()
        self.weight = torch.nn.Parameter(torch.full((num_parameters,), init, dtype=dtype, device=device))

    def forward(self, x):
        a = self.weight
        if a.numel() > 1:
            a = a.reshape(1, -1, *([1] * (x.dim() - 2)))
        pos = _ew.unary("relu", x)
        neg = _ew.binary("sub", x, pos)
        return _ew.binary("add", pos, _ew.binary("mul", a.to(x.dtype), neg))


class RReLU(Module):
    """Randomised leaky ReLU.  Training: negative slopes ~ U(lower, upper), one per element
    (PyTorch's rule, the default) or one per call with ``per_element=False`` (the reference's
    rule, nn/activation.go:300-304); eval: the midpoint slope.  ``Seed`` makes the draws
    reproducible (nn/activation.go:297)."""

    def __init__(self, lower: float = 1.0 / 8, upper: float = 1.0 / 3, per_element: bool = True):
        super().__init__()
        self.lower, self.upper, self.per_element = lower, upper, per_element
        self._gen = None

    def Seed(self, seed: int) -> "RReLU":
        self._seed = int(seed)
        self._gen = None
        return self

    def _generator(self, device):
        if getattr(self, "_seed", None) is None:
            return None
        if self._gen is None or self._gen.device != device:
            self._gen = torch.Generator(device=device).manual_seed(self._seed)
        return self._gen

    def forward(self, x):
        if self.training:
            g = self._generator(x.device)
            if not self.per_element:
                u = torch.rand((), generator=self._generator(torch.device("cpu"))).item()
                return _ew.unary("leakyrelu", x, self.lower + u * (self.upper - self.lower))
            slope = torch.empty_like(x).uniform_(self.lower, self.upper, generator=g)
            return torch.where(x >= 0, x, x * slope)
        return _ew.unary("leakyrelu", x, (self.lower + self.upper) / 2)


RReLULayer = RReLU


class GLU(Module):
    """a * sigmoid(b) where (a, b) split ``dim`` in halves."""

    def __init__(self, dim: int = -1):
        super().__init__()
        self.dim = dim

    def forward(self, x):
        a, b = x.chunk(2, dim=self.dim)
        return _ew.binary("mul", a.contiguous(), _ew.unary("sigmoid", b.contiguous()))

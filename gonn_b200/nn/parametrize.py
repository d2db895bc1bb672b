"""Weight reparametrizations (nn/parametrize.go:79-475, nn/parametrize_generic.go:57-581).

* ``WeightNormLinear`` / ``WeightNormConv2d``: parameters ``weight_g`` (per-output-row norm)
  and ``weight_v``; effective weight g * v / ||v||_row; ``Remove*`` bakes it into a fresh layer.
* ``SpectralNormLinear`` / ``SpectralNormConv2d``: parameter ``weight_orig``, buffers ``u``,
  ``v``; 15 warm-up power iterations at construction, ``n_power_iterations`` (default 1) per
  training forward, eps 1e-12; sigma = u^T W v is differentiable in W with u, v constant.
* Generic: ``ParametrizedLinear`` / ``ParametrizedConv2d`` own ``weight_orig`` (and
  ``bias_orig``) and apply a chain of shape-preserving functions in registration order;
  ``RightInverse`` gives function-preserving initialisation and ``SetEffectiveWeight``;
  ``Cached`` evaluates the chain once for several forwards.
"""
from __future__ import annotations

import contextlib
import copy
from typing import Callable, List, Optional

import torch

from .conv import Conv2d
from .linear import Linear
from .module import Module


def _run_with_weight(layer, x, w, b):
    """Forward of ``layer`` with the given weight / bias tensors (differentiable in both)."""
    params = {"weight": w}
    if b is not None:
        params["bias"] = b
    return torch.func.functional_call(layer, params, (x,))


def _row_norm(v):
    return v.reshape(v.shape[0], -1).norm(dim=1).reshape(-1, *([1] * (v.dim() - 1)))


class _WeightNorm(Module):
    def __init__(self, layer):
        super().__init__()
        self._layer = [layer]            # not a child: its own weight is replaced
        w = layer.weight.detach()
        self.weight_g = torch.nn.Parameter(_row_norm(w).clone())
        self.weight_v = torch.nn.Parameter(w.clone())
        self.bias = layer.bias

    def EffectiveWeight(self):
        return self.weight_g * self.weight_v / _row_norm(self.weight_v)

    def forward(self, x):
        return _run_with_weight(self._layer[0], x, self.EffectiveWeight(), self.bias)


class WeightNormLinear(_WeightNorm):
    pass


class WeightNormConv2d(_WeightNorm):
    pass


def _bake(wrapper, w):
    """A fresh plain layer holding ``w`` (and a copy of the bias); the wrapper and the layer it
    wraps are left as they are (nn/parametrize.go:140-155, 391-401)."""
    layer = copy.deepcopy(wrapper._layer[0])
    with torch.no_grad():
        layer.weight.copy_(w)
    return layer


def RemoveWeightNormLinear(m: WeightNormLinear) -> Linear:
    return _bake(m, m.EffectiveWeight().detach())


def RemoveWeightNormConv2d(m: WeightNormConv2d) -> Conv2d:
    return _bake(m, m.EffectiveWeight().detach())


def _l2n(x, eps):
    return x / (x.norm() + eps)


class _SpectralNorm(Module):
    def __init__(self, layer, n_power_iterations: int = 1, eps: float = 1e-12):
        super().__init__()
        self._layer = [layer]
        self.n_power_iterations, self.eps = n_power_iterations, eps
        self.weight_orig = layer.weight         # the same tensor object as the wrapped layer's
        self.bias = layer.bias
        w2 = self._mat().detach()
        m, n = w2.shape
        u = _l2n(torch.randn(m, dtype=w2.dtype, device=w2.device), eps)
        v = _l2n(torch.randn(n, dtype=w2.dtype, device=w2.device), eps)
        self.register_buffer("u", u)
        self.register_buffer("v", v)
        self._power(15)

    def _mat(self):
        return self.weight_orig.reshape(self.weight_orig.shape[0], -1)

    @torch.no_grad()
    def _power(self, iters):
        w = self._mat().detach()
        for _ in range(iters):
            self.v.copy_(_l2n(w.t() @ self.u, self.eps))
            self.u.copy_(_l2n(w @ self.v, self.eps))

    def EstimatedSigma(self) -> float:
        return float(self.u @ (self._mat().detach() @ self.v))

    def EffectiveWeight(self):
        sigma = self.u @ (self._mat() @ self.v)
        return self.weight_orig / sigma

    def forward(self, x):
        if self.training:
            self._power(self.n_power_iterations)
        return _run_with_weight(self._layer[0], x, self.EffectiveWeight(), self.bias)


class SpectralNormLinear(_SpectralNorm):
    pass


class SpectralNormConv2d(_SpectralNorm):
    pass


def RemoveSpectralNormLinear(m) -> Linear:
    return _bake(m, m.EffectiveWeight().detach())


def RemoveSpectralNormConv2d(m) -> Conv2d:
    return _bake(m, m.EffectiveWeight().detach())


# ---- generic parametrizations ---------------------------------------------------------------
class Parametrization:
    """``Apply(orig) -> effective`` (shape preserving)."""

    def Apply(self, orig):
        raise NotImplementedError


class ParametrizationFunc(Parametrization):
    def __init__(self, fn: Callable):
        self.fn = fn

    def Apply(self, orig):
        return self.fn(orig)


class InvertibleParametrization(Parametrization):
    """Adds ``RightInverse(value) -> orig`` with Apply(RightInverse(v)) == v."""

    def __init__(self, fwd: Callable, inv: Callable):
        self.Fwd, self.Inv = fwd, inv

    def Apply(self, orig):
        return self.Fwd(orig)

    def RightInverse(self, v):
        return self.Inv(v)


# the reference's name for the same contract (nn/parametrize_generic.go:57-80)
ParametrizationWithInverse = InvertibleParametrization


def _as_param(p):
    return p if isinstance(p, Parametrization) else ParametrizationFunc(p)


class _Parametrized(Module):
    def __init__(self, layer, weight_p, bias_p=None):
        super().__init__()
        self._layer = [layer]
        self._wchain: List[Parametrization] = []
        self._bchain: List[Parametrization] = []
        self._cache = None
        self.weight_orig = torch.nn.Parameter(layer.weight.detach().clone())
        self.bias_orig = None
        self.bias = layer.bias
        self.AddParametrization(weight_p)
        if bias_p is not None and layer.bias is not None:
            bp = _as_param(bias_p)
            init = bp.RightInverse(layer.bias.detach()) if hasattr(bp, "RightInverse") else layer.bias.detach()
            self.bias_orig = torch.nn.Parameter(init.clone())
            self.bias = None
            self._bchain.append(bp)

    def AddParametrization(self, p):
        p = _as_param(p)
        if hasattr(p, "RightInverse") and not self._wchain:
            # function-preserving start: orig = RightInverse(current effective weight)
            with torch.no_grad():
                self.weight_orig.copy_(p.RightInverse(self.weight_orig.detach()))
        out = p.Apply(self._apply(self._wchain, self.weight_orig))
        if tuple(out.shape) != tuple(self.weight_orig.shape):
            raise ValueError("parametrization must preserve the shape")
        self._wchain.append(p)
        return self

    @staticmethod
    def _apply(chain, t):
        for p in chain:
            t = p.Apply(t)
        return t

    def EffectiveWeight(self):
        if self._cache is not None:
            return self._cache[0]
        return self._apply(self._wchain, self.weight_orig)

    def EffectiveBias(self):
        if self.bias_orig is None:
            return self.bias
        if self._cache is not None:
            return self._cache[1]
        return self._apply(self._bchain, self.bias_orig)

    def SetEffectiveWeight(self, value):
        """Sets weight_orig so that the effective weight equals ``value`` (needs RightInverse on
        every parametrization of the chain)."""
        v = value.detach()
        for p in reversed(self._wchain):
            if not hasattr(p, "RightInverse"):
                raise ValueError("SetEffectiveWeight: a parametrization has no RightInverse")
            v = p.RightInverse(v)
        with torch.no_grad():
            self.weight_orig.copy_(v)

    @contextlib.contextmanager
    def Cached(self):
        """Within the block the chain is evaluated once and reused by every forward."""
        self._cache = (self._apply(self._wchain, self.weight_orig),
                       self._apply(self._bchain, self.bias_orig) if self.bias_orig is not None else None)
        try:
            yield self
        finally:
            self._cache = None

    def forward(self, x):
        return _run_with_weight(self._layer[0], x, self.EffectiveWeight(), self.EffectiveBias())


class ParametrizedLinear(_Parametrized):
    pass


class ParametrizedConv2d(_Parametrized):
    pass


def IsParametrized(m) -> bool:
    return isinstance(m, (_Parametrized, _WeightNorm, _SpectralNorm))


@contextlib.contextmanager
def ParametrizeCachedAll(*modules):
    with contextlib.ExitStack() as st:
        for m in modules:
            st.enter_context(m.Cached())
        yield


def RemoveParametrizations(m, leave_parametrized: bool = True):
    """Returns the plain layer; with ``leave_parametrized`` its weight is the current effective
    weight, otherwise the raw ``weight_orig``."""
    layer = m._layer[0]
    with torch.no_grad():
        layer.weight.copy_(m.EffectiveWeight().detach() if leave_parametrized else m.weight_orig.detach())
        if getattr(m, "bias_orig", None) is not None:
            layer.bias.copy_(m.EffectiveBias().detach() if leave_parametrized else m.bias_orig.detach())
    return layer


RemoveParametrizationsLinear = RemoveParametrizations
RemoveParametrizationsConv2d = RemoveParametrizations

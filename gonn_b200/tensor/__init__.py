"""Tensor API with the reference's vocabulary over ``torch.Tensor``.

Storage, strides and the autograd tape are PyTorch's; the functions here give the
reference's operation set (tensor/*.go) names and semantics, and route the math to
the native kernels for CUDA tensors:

* constructors ``New, NewLike, Zeros, Ones, Full, Randn, Uniform, Arange, Eye, Scalar``
* the unary-op registry ``RegisterUnary / LookupUnary / UnaryOpNames / Unary`` with the
  25 built-in names, plus the parameterised ops (``Pow, Clip, LeakyReLU, ELU, ...``)
* broadcasting binary ops, ``MatMul`` / ``BMM``, reductions, shape / index / extra ops
* dtype helpers ``AsType`` / ``To`` and the rounding emulation ``RoundTo``
* the dispatch policy (``SetDispatchPolicy``), kept for API parity: CUDA tensors
  always run on kernels, CPU tensors always on the host path.
"""
from .api import *  # noqa: F401,F403
from .api import __all__  # noqa: F401

from . import api as _api, methods as _methods

_methods.install(_api)          # x.Add(y).ReLU().Sum(): the reference's method spellings

"""Method spellings of the tensor operations.

The reference's operations are methods on its tensor (``x.Add(y).ReLU().Sum()``,
tensor/*.go); here they are functions of this package over ``torch.Tensor``.  ``install()``
also attaches every one of them to ``torch.Tensor`` under the reference's capitalised name, so
chained code reads the same.  Only names that ``torch.Tensor`` does not already define are
added (``T`` stays torch's transpose property: write ``x.Transpose()`` or ``x.T``, not ``x.T()``), and
nothing lower-case is touched.  Importing ``gonn_b200.tensor`` installs them once.
"""
from __future__ import annotations

import torch

METHOD_NAMES = (
    "Abs Add AddScalar ArgMax ArgMin ArgWhere AsType BMM Backward CELU Chunk Clip Copy Cos Cumsum Div DivScalar "
    "ELU Exp Expand Flatten Flip GELU GELUExact Gather HardSigmoid HardSwish HardTanh Hardshrink IndexSelect Item "
    "LeakyReLU Log LogSigmoid LogSoftmax MaskedFill MatMul Max MaxAxis Mean MeanAxis Min MinAxis Mish Mul MulScalar "
    "Neg Numel Permute Pow RReLU ReLU ReLU6 Reciprocal Repeat Reshape SELU SetRequiresGrad SiLU Sigmoid Sin Softmax "
    "Softplus SoftplusBeta Softshrink Softsign Split Sqrt Square Squeeze String Sub SubScalar Sum SumAxis Swish Tan "
    "Tanh Tanhshrink Threshold Tile To Transpose Tril Triu Unary Unsqueeze View ZeroGrad").split()

_installed = []


def install(namespace) -> list:
    """Attaches ``namespace.<Name>`` as ``torch.Tensor.<Name>`` for every name above that
    torch does not define; returns the names added (empty on a second call)."""
    added = []
    for name in METHOD_NAMES:
        fn = getattr(namespace, name, None)
        if fn is None or hasattr(torch.Tensor, name):
            continue
        setattr(torch.Tensor, name, fn)       # a plain function: ``self`` binds to the first argument
        added.append(name)
    for name, fn in (("Dim", lambda self: self.dim()), ("DType", lambda self: self.dtype)):
        if not hasattr(torch.Tensor, name):
            setattr(torch.Tensor, name, fn)
            added.append(name)
    # exported fields of the reference's tensor (tensor/tensor.go:14-30) as properties: the values in
    # row-major order, the shape as a list, the gradient (assignable) and the gradient flag
    fields = {
        "Data": property(lambda self: self.detach().reshape(-1)),
        "Shape": property(lambda self: list(self.shape)),
        "Grad": property(lambda self: self.grad, lambda self, g: setattr(self, "grad", g)),
        "RequiresGrad": property(lambda self: self.requires_grad),
    }
    for name, prop in fields.items():
        if not hasattr(torch.Tensor, name):
            setattr(torch.Tensor, name, prop)
            added.append(name)
    _installed.extend(added)
    return added


def installed() -> list:
    return list(_installed)

"""Linear family (nn/linear.go:11-207): Linear, Bilinear."""
from __future__ import annotations

import torch

from ..ops.linear import linear as _linear, matmul as _matmul
from .init import fan_in_uniform_
from .module import Module


class Linear(Module):
    """``y = x W^T + b`` with W of shape (out, in); leading dims are flattened.

    ``activation`` ("relu", "gelu", "geluexact") fuses the activation into the GEMM
    epilogue; the default keeps the reference's plain affine map.
    """

    def __init__(self, in_features: int, out_features: int, bias: bool = True, *, activation=None,
                 dtype=torch.float32, device=None):
        super().__init__()
        self.in_features, self.out_features, self.activation = in_features, out_features, activation
        self.weight = torch.nn.Parameter(torch.empty(out_features, in_features, dtype=dtype, device=device))
        self.bias = torch.nn.Parameter(torch.empty(out_features, dtype=dtype, device=device)) if bias else None
        fan_in_uniform_(self.weight.data, self.bias.data if bias else None, in_features)

    def forward(self, x, residual=None, bias_grad: bool = True):
        if x.shape[-1] != self.in_features:
            raise ValueError(f"nn.Linear: expected last dim {self.in_features}, got {x.shape[-1]}")
        return _linear(x, self.weight, self.bias, self.activation, residual, bias_grad)

    def extra_repr(self):
        return f"{self.in_features}, {self.out_features}, bias={self.bias is not None}"


class Bilinear(Module):
    """``y_k = x1^T W_k x2 + b_k`` with W of shape (out, in1, in2)."""

    def __init__(self, in1: int, in2: int, out_features: int, bias: bool = True, *, dtype=torch.float32,
                 device=None):
        super().__init__()
        self.in1, self.in2, self.out_features = in1, in2, out_features
        self.weight = torch.nn.Parameter(torch.empty(out_features, in1, in2, dtype=dtype, device=device))
        self.bias = torch.nn.Parameter(torch.empty(out_features, dtype=dtype, device=device)) if bias else None
        fan_in_uniform_(self.weight.data, self.bias.data if bias else None, in1)

    def forward(self, x1, x2):
        lead = x1.shape[:-1]
        a = x1.reshape(-1, self.in1)
        b = x2.reshape(-1, self.in2)
        # t[n, k*in2 + j] = sum_i a[n,i] W[k,i,j]
        w2 = self.weight.permute(1, 0, 2).reshape(self.in1, self.out_features * self.in2)
        t = _matmul(a, w2).reshape(-1, self.out_features, self.in2)
        y = (t * b[:, None, :]).sum(-1)
        if self.bias is not None:
            y = y + self.bias
        return y.reshape(*lead, self.out_features)

"""MLP classifier: Linear -> ReLU -> ... -> Linear (the quick-start model family of the
reference's README and examples/mlp)."""
from __future__ import annotations

from typing import Sequence

import torch

from ..nn.activation import ReLU
from ..nn.linear import Linear
from ..nn.module import Flatten, Module, Sequential


class MLP(Module):
    def __init__(self, sizes: Sequence[int] = (784, 256, 128, 10), *, dtype=torch.float32, device=None,
                 fuse_activation: bool = False):
        super().__init__()
        layers = [Flatten()]
        for i in range(len(sizes) - 1):
            last = i == len(sizes) - 2
            if fuse_activation and not last:
                layers.append(Linear(sizes[i], sizes[i + 1], activation="relu", dtype=dtype, device=device))
            else:
                layers.append(Linear(sizes[i], sizes[i + 1], dtype=dtype, device=device))
                if not last:
                    layers.append(ReLU())
        self.net = Sequential(*layers)

    def forward(self, x):
        return self.net(x)

"""Small CNN: Conv 3->64 3x3, BatchNorm, ReLU, MaxPool 2, Conv 64->128 3x3, BatchNorm, ReLU,
global average pool, Linear 128->10 (3x32x32 inputs).

The layer sequence of the reference's convolutional example (examples/cnn/main.go:32-37: convolution,
normalisation, ReLU, pooling, a linear head) at the width of the data-parallel benchmark configuration;
the reference runs every convolution as a gather + GEMM on the host (nn/conv.go:341-380), here they
are implicit-GEMM kernels."""
from __future__ import annotations

import torch

from ..nn.batchnorm import BatchNorm2d
from ..nn.conv import Conv2d
from ..nn.linear import Linear
from ..nn.module import Module
from ..nn.pool import AdaptiveAvgPool2d, MaxPool2d
from ..ops.softmax import cross_entropy


class SmallCNN(Module):
    def __init__(self, num_classes: int = 10, sync_bn: bool = False, group=None, *, dtype=torch.float32,
                 device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        if sync_bn:
            from ..distributed.syncbn import SyncBatchNorm2d

            def BN(c):
                return SyncBatchNorm2d(c, group=group, fused_relu=True, **kw)
        else:
            def BN(c):
                return BatchNorm2d(c, fused_relu=True, **kw)
        self.conv1 = Conv2d(3, 64, 3, **kw)
        self.bn1 = BN(64)
        self.pool = MaxPool2d(2)
        self.conv2 = Conv2d(64, 128, 3, **kw)
        self.bn2 = BN(128)
        self.gap = AdaptiveAvgPool2d(1)
        self.fc = Linear(128, num_classes, **kw)

    def forward(self, x):
        x = self.pool(self.bn1(self.conv1(x)))      # ReLU is fused into the BatchNorm kernel
        x = self.gap(self.bn2(self.conv2(x)))
        return self.fc(x.flatten(1))

    def loss(self, x, y):
        return cross_entropy(self.forward(x), y)

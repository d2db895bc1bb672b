"""AdaptiveLogSoftmaxWithLoss (nn/adaptive_softmax.go:38-215): a head over the shortlist plus
one logit per cluster, and per-cluster tails of two bias-free Linears with a bottleneck of
floor(in / div^(i+1)) >= 1 units.  Children ``head``, ``tail.i``."""
from __future__ import annotations

from typing import Sequence

import torch

from .linear import Linear
from .module import Module, ModuleList, Sequential


class AdaptiveLogSoftmaxWithLoss(Module):
    def __init__(self, in_features: int, n_classes: int, cutoffs: Sequence[int], div_value: float = 4.0,
                 head_bias: bool = False, *, dtype=torch.float32, device=None):
        super().__init__()
        cutoffs = list(cutoffs)
        if cutoffs != sorted(set(cutoffs)) or not cutoffs or cutoffs[0] <= 0 or cutoffs[-1] >= n_classes:
            raise ValueError("AdaptiveLogSoftmaxWithLoss: cutoffs must be unique, increasing, in (0, n_classes)")
        self.in_features, self.n_classes, self.div_value = in_features, n_classes, div_value
        self.cutoffs = cutoffs + [n_classes]
        self.shortlist = self.cutoffs[0]
        self.n_clusters = len(self.cutoffs) - 1
        kw = dict(dtype=dtype, device=device)
        self.head = Linear(in_features, self.shortlist + self.n_clusters, head_bias, **kw)
        tails = []
        for i in range(self.n_clusters):
            hid = max(int(in_features // (div_value ** (i + 1))), 1)
            osz = self.cutoffs[i + 1] - self.cutoffs[i]
            tails.append(Sequential(Linear(in_features, hid, False, **kw), Linear(hid, osz, False, **kw)))
        self.tail = ModuleList(tails)

    def LogProb(self, x):
        """Full (N, n_classes) log-probabilities."""
        ct = torch.float64 if x.dtype == torch.float64 else torch.float32     # 16-bit inputs widen to fp32
        head_lp = torch.log_softmax(self.head(x).to(ct), 1)
        out = [head_lp[:, :self.shortlist]]
        for i in range(self.n_clusters):
            tl = torch.log_softmax(self.tail[i](x).to(ct), 1)
            out.append(tl + head_lp[:, self.shortlist + i:self.shortlist + i + 1])
        return torch.cat(out, 1)

    def forward(self, x, target):
        """Returns (per-sample target log-probability, mean negative log-likelihood)."""
        lp = self.LogProb(x)
        out = lp.gather(1, target.long()[:, None]).squeeze(1)
        return out, -out.mean()

    def Predict(self, x):
        return self.LogProb(x).argmax(1)

"""Loss functions (nn/loss.go:16-480, nn/ctc.go:40-229).

All take ``reduction`` = "mean" (default) | "sum" | "none".  Class-index losses
also take ``weight`` (per-class), ``ignore_index`` and (cross-entropy only)
``label_smoothing``; their mean divides by the summed weights of the non-ignored
targets.  CrossEntropyLoss runs the fused kernel on CUDA; the other losses are
compositions of differentiable tensor ops with the reference's exact formulas
(clamps, eps values and all).
"""
from __future__ import annotations

import math
from typing import Callable, Optional

import torch

from ..ops.softmax import cross_entropy as _cross_entropy
from .module import Module

INF = float("inf")


def _reduce(t: torch.Tensor, reduction: str) -> torch.Tensor:
    if reduction == "mean":
        return t.mean()
    if reduction == "sum":
        return t.sum()
    if reduction == "none":
        return t
    raise ValueError(f"unknown reduction {reduction!r}")


def MSELoss(pred, target, reduction="mean"):
    return _reduce((pred - target) ** 2, reduction)


def MAELoss(pred, target, reduction="mean"):
    return _reduce((pred - target).abs(), reduction)


L1Loss = MAELoss


def HuberLoss(pred, target, delta: float = 1.0, reduction="mean"):
    """0.5 d^2 for |d| <= delta, delta (|d| - 0.5 delta) beyond."""
    d = (pred - target).abs()
    quad = torch.clamp(d, max=delta)
    return _reduce(0.5 * quad * quad + delta * (d - quad), reduction)


def SmoothL1Loss(pred, target, beta: float = 1.0, reduction="mean"):
    """Identical to HuberLoss with delta = beta (the reference's definition)."""
    return HuberLoss(pred, target, beta, reduction)


def CrossEntropyLoss(logits, targets, weight=None, ignore_index: Optional[int] = None,
                     label_smoothing: float = 0.0, reduction="mean"):
    """NLL of log-softmax over (N, C) logits and (N,) class indices."""
    if logits.dim() != 2:
        raise ValueError("CrossEntropyLoss: input must be 2D (N, C)")
    if targets.numel() != logits.shape[0]:
        raise ValueError("CrossEntropyLoss: targets must have N entries")
    return _cross_entropy(logits, targets, weight, ignore_index, label_smoothing, reduction)


def NLLLoss(log_probs, targets, weight=None, ignore_index: Optional[int] = None, reduction="mean"):
    """-w[y] * logP[n, y]; ignored rows contribute 0; mean divides by the summed weights."""
    if log_probs.dim() != 2:
        raise ValueError("NLLLoss: input must be 2D (N, C)")
    N, C = log_probs.shape
    t = targets.long().reshape(-1)
    if t.numel() != N:
        raise ValueError("NLLLoss: targets must have N entries")
    keep = torch.ones(N, dtype=log_probs.dtype, device=log_probs.device)
    if ignore_index is not None:
        keep = (t != ignore_index).to(log_probs.dtype)
    safe = torch.where(keep.bool(), t, torch.zeros_like(t))
    if bool(((safe < 0) | (safe >= C)).any()):
        raise ValueError("NLLLoss: target out of range")
    w = keep if weight is None else weight.to(log_probs.dtype)[safe] * keep
    vec = -(log_probs.gather(1, safe[:, None]).squeeze(1)) * w
    if reduction == "sum":
        return vec.sum()
    if reduction == "none":
        return vec
    return vec.sum() / w.sum()


def BCELoss(pred, target, reduction="mean"):
    eps = 1e-12
    p = torch.clamp(pred, eps, 1 - eps)
    return _reduce(-(target * p.log() + (1 - target) * (1 - p).log()), reduction)


def BCEWithLogitsLoss(logits, target, reduction="mean"):
    """max(z,0) - z t + log(1 + exp(-|z|))."""
    return _reduce(torch.relu(logits) - logits * target + torch.nn.functional.softplus(-logits.abs()), reduction)


def KLDivLoss(input, target, reduction="mean"):
    """input: log-probabilities, target: probabilities; target * (log target - input)."""
    return _reduce(target * (torch.clamp(target, min=1e-12).log() - input), reduction)


def PoissonNLLLoss(input, target, log_input: bool = True, reduction="mean"):
    if log_input:
        return _reduce(input.exp() - target * input, reduction)
    return _reduce(input - target * (input + 1e-8).log(), reduction)


def GaussianNLLLoss(input, target, var, reduction="mean"):
    return _reduce(0.5 * (var.log() + (input - target) ** 2 / var), reduction)


def MarginRankingLoss(x1, x2, y, margin: float = 0.0, reduction="mean"):
    return _reduce(torch.clamp(-y * (x1 - x2) + margin, min=0), reduction)


def HingeEmbeddingLoss(x, y, margin: float = 1.0, reduction="mean"):
    pos, neg = (y + 1) * 0.5, (1 - y) * 0.5
    return _reduce(pos * x + neg * torch.clamp(margin - x, min=0), reduction)


def CosineEmbeddingLoss(x1, x2, y, margin: float = 0.0, reduction="mean"):
    eps = 1e-8
    cs = (x1 * x2).sum(1) / (((x1 * x1).sum(1) + eps).sqrt() * ((x2 * x2).sum(1) + eps).sqrt())
    pos, neg = (y + 1) * 0.5, (1 - y) * 0.5
    return _reduce(pos * (1 - cs) + neg * torch.clamp(cs - margin, min=0), reduction)


def PairwiseL2Distance(x1, x2):
    return (((x1 - x2) ** 2).sum(1) + 1e-8).sqrt()


def TripletMarginLoss(anchor, positive, negative, margin: float = 1.0, reduction="mean"):
    return _reduce(torch.clamp(PairwiseL2Distance(anchor, positive) - PairwiseL2Distance(anchor, negative) + margin,
                               min=0), reduction)


def TripletMarginWithDistanceLoss(anchor, positive, negative, distance: Optional[Callable] = None,
                                  margin: float = 1.0, reduction="mean"):
    distance = distance or PairwiseL2Distance
    return _reduce(torch.clamp(distance(anchor, positive) - distance(anchor, negative) + margin, min=0), reduction)


def MultiMarginLoss(input, target, margin: float = 1.0, reduction="mean"):
    if input.dim() != 2:
        raise ValueError("MultiMarginLoss: input must be 2D (N, C)")
    N, C = input.shape
    t = target.long().reshape(-1)
    if bool(((t < 0) | (t >= C)).any()):
        raise ValueError("MultiMarginLoss: target out of range")
    xt = input.gather(1, t[:, None])
    m = torch.clamp(input - xt + margin, min=0)
    mask = torch.ones_like(m).scatter_(1, t[:, None], 0.0)
    return _reduce((m * mask).sum(1) / (C - 1), reduction)


def SoftMarginLoss(x, y, reduction="mean"):
    return _reduce(torch.nn.functional.softplus(-y * x), reduction)


def MultiLabelSoftMarginLoss(x, y, reduction="mean"):
    if x.dim() != 2:
        raise ValueError("MultiLabelSoftMarginLoss: input must be 2D (N, C)")
    per = torch.relu(x) - x * y + torch.nn.functional.softplus(-x.abs())
    return _reduce(per.mean(1), reduction)


def MultiLabelMarginLoss(x, y, reduction="mean"):
    """Targets: class indices per row, terminated by the first negative entry."""
    if x.dim() == 1:
        x, y = x[None], y[None]
    if x.dim() != 2 or tuple(y.shape) != tuple(x.shape):
        raise ValueError("MultiLabelMarginLoss: target must have the same shape as input")
    N, C = x.shape
    out = []
    for n in range(N):
        tgt = []
        for c in range(C):
            v = int(y[n, c])
            if v < 0:
                break
            if v >= C:
                raise ValueError("MultiLabelMarginLoss: target class out of range")
            tgt.append(v)
        if not tgt:
            out.append(x.new_zeros(()))
            continue
        ti = torch.tensor(tgt, device=x.device)
        hinge = torch.clamp(x[n][None, :] - x[n][ti][:, None] + 1, min=0)
        mask = torch.ones(C, dtype=x.dtype, device=x.device)
        mask[ti] = 0
        out.append((hinge * mask).sum() / C)
    return _reduce(torch.stack(out), reduction)


def CTCLoss(log_probs, targets, input_lengths, target_lengths, blank: int = 0, reduction="mean"):
    """Connectionist temporal classification (nn/ctc.go:40-229).

    ``log_probs``: (T, N, C) log-softmax outputs; ``targets``: (N, S) padded class indices;
    lengths: per-sample.  Log-space alpha recursion over the blank-interleaved sequence
    (length 2S+1); a skip is allowed only onto a label that differs from the one two states
    back; loss = -logaddexp(last two states).  An infeasible alignment gives +inf loss and a
    zero gradient.  ``mean`` divides each sample by max(target_len, 1), then averages.
    """
    T, N, C = log_probs.shape
    losses = []
    neg_inf = torch.tensor(-INF, dtype=log_probs.dtype, device=log_probs.device)
    for n in range(N):
        Tn, Sn = int(input_lengths[n]), int(target_lengths[n])
        lab = [int(v) for v in targets[n, :Sn]]
        ext = [blank]
        for l in lab:
            ext += [l, blank]
        L = len(ext)
        lp = log_probs[:Tn, n, :]
        alpha = [neg_inf] * L
        alpha[0] = lp[0, ext[0]]
        if L > 1:
            alpha[1] = lp[0, ext[1]]
        for t in range(1, Tn):
            new = []
            for s in range(L):
                terms = [alpha[s]]
                if s >= 1:
                    terms.append(alpha[s - 1])
                if s >= 2 and ext[s] != blank and ext[s] != ext[s - 2]:
                    terms.append(alpha[s - 2])
                st = torch.stack(terms)
                m = st.max()
                if torch.isinf(m) and m < 0:
                    new.append(neg_inf)
                else:
                    new.append(m + torch.log(torch.exp(st - m).sum()) + lp[t, ext[s]])
            alpha = new
        tail = torch.stack([alpha[L - 1]] + ([alpha[L - 2]] if L > 1 else []))
        m = tail.max()
        if torch.isinf(m) and m < 0:
            losses.append((log_probs.sum() * 0) + INF)  # infeasible: +inf loss, zero gradient
        else:
            losses.append(-(m + torch.log(torch.exp(tail - m).sum())))
    vec = torch.stack(losses)
    if reduction == "none":
        return vec
    if reduction == "sum":
        return vec.sum()
    tl = torch.as_tensor([max(int(v), 1) for v in target_lengths], dtype=vec.dtype, device=vec.device)
    return (vec / tl).mean()


class _LossModule(Module):
    fn: Callable = None

    def __init__(self, **kw):
        super().__init__()
        self.kw = kw

    def forward(self, *a):
        return type(self).fn(*a, **self.kw)


def _loss_module(fn):
    return type(fn.__name__ + "Module", (_LossModule,), {"fn": staticmethod(fn), "__doc__": fn.__doc__})


CrossEntropy = _loss_module(CrossEntropyLoss)
MSE = _loss_module(MSELoss)

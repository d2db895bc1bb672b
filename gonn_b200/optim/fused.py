"""Kernel-backed optimizers: SGD, Adam, AdamW, Lion, LAMB.

Update rules are the reference's (optim/sgd.go:47-69, adam.go:61-77,
adamw.go:64-84, lion.go:61-76, lamb.go:73-108); on CUDA each parameter group
is updated by multi-tensor kernel launches, on CPU by the same formulas as
tensor expressions.  State buffer names: ``momentum_buf``; ``m``, ``v``.
"""
from __future__ import annotations

import math
from typing import List

import torch

from ..ops import multi_tensor as mt
from .base import Group, Optimizer, as_groups, state_dtype


class SGD(Optimizer):
    """v = mu*v + g; p -= lr*v (Nesterov: p -= lr*(g + mu*v)); coupled weight decay."""

    def __init__(self, params, lr: float = 0.01, momentum: float = 0.0, nesterov: bool = False,
                 weight_decay: float = 0.0):
        super().__init__(as_groups(params, lr, weight_decay))
        self.momentum, self.nesterov = momentum, nesterov

    def _update(self, g: Group, params: List[torch.Tensor]):
        for ps in mt.by_dtype(params):
            bufs = [self.state(p).buf("momentum_buf", p, state_dtype(p)) for p in ps] if self.momentum else None
            if mt.native(ps[0]):
                masters = [self.master(p) for p in ps]
                flags = (1 if self.nesterov else 0) | (4 if self.momentum else 0)
                mt.launch(mt.SGD, ps, [p.grad for p in ps], masters, bufs, None,
                          [g.lr, g.weight_decay, 0, 0, 0, 1, 1, self.momentum, 1.0], flags)
                continue
            for i, p in enumerate(ps):
                gr = p.grad.to(state_dtype(p))
                pv = p.data.to(state_dtype(p))
                if g.weight_decay:
                    gr = gr + g.weight_decay * pv
                if self.momentum:
                    v = bufs[i]
                    v.mul_(self.momentum).add_(gr)
                    upd = gr + self.momentum * v if self.nesterov else v
                else:
                    upd = gr
                if pv is p.data or pv.data_ptr() == p.data.data_ptr():
                    p.data.sub_(upd * g.lr)          # same dtype: update in place, one temporary
                else:
                    p.data.copy_((pv - g.lr * upd).to(p.dtype))


class Adam(Optimizer):
    """Adam with one shared step counter; weight decay is coupled (added to the gradient)."""

    decoupled = False

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.0):
        super().__init__(as_groups(params, lr, weight_decay))
        self.beta1, self.beta2 = betas
        self.eps = eps
        self.t = 0

    def _begin_step(self):
        self.t += 1

    def _extra_scalars(self):
        return {"t": self.t}

    def _load_extra_scalars(self, d):
        self.t = int(d.get("t", 0))

    def _update(self, g: Group, params: List[torch.Tensor]):
        bc1 = 1 - self.beta1 ** self.t
        bc2 = 1 - self.beta2 ** self.t
        for ps in mt.by_dtype(params):
            ms = [self.state(p).buf("m", p, state_dtype(p)) for p in ps]
            vs = [self.state(p).buf("v", p, state_dtype(p)) for p in ps]
            if mt.native(ps[0]):
                masters = [self.master(p) for p in ps]
                mt.launch(mt.ADAM, ps, [p.grad for p in ps], masters, ms, vs,
                          [g.lr, g.weight_decay, self.beta1, self.beta2, self.eps, bc1, bc2, 0, 1.0],
                          2 if self.decoupled else 0)
                continue
            for p, m, v in zip(ps, ms, vs):
                ct = state_dtype(p)
                gr, pv = p.grad.to(ct), p.data.to(ct)
                if g.weight_decay:
                    if self.decoupled:
                        pv = pv - g.lr * g.weight_decay * pv
                    else:
                        gr = gr + g.weight_decay * pv
                m.mul_(self.beta1).add_(gr, alpha=1 - self.beta1)
                v.mul_(self.beta2).addcmul_(gr, gr, value=1 - self.beta2)
                pv = pv - g.lr * (m / bc1) / ((v / bc2).sqrt() + self.eps)
                p.data.copy_(pv.to(p.dtype))


class AdamW(Adam):
    """Adam with decoupled decay ``p -= lr*wd*p`` applied before the Adam term.  The
    single-list constructor defaults to weight_decay 0.01; groups keep their own values."""

    decoupled = True

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.01):
        super().__init__(params, lr, betas, eps, weight_decay)


class Lion(Optimizer):
    def __init__(self, params, lr: float = 1e-4, betas=(0.9, 0.99), weight_decay: float = 0.0):
        super().__init__(as_groups(params, lr, weight_decay))
        self.beta1, self.beta2 = betas

    def _update(self, g: Group, params: List[torch.Tensor]):
        for ps in mt.by_dtype(params):
            ms = [self.state(p).buf("m", p, state_dtype(p)) for p in ps]
            if mt.native(ps[0]):
                mt.launch(mt.LION, ps, [p.grad for p in ps], [self.master(p) for p in ps], ms, None,
                          [g.lr, g.weight_decay, self.beta1, self.beta2, 0, 1, 1, 0, 1.0], 0)
                continue
            for p, m in zip(ps, ms):
                ct = state_dtype(p)
                gr, pv = p.grad.to(ct), p.data.to(ct)
                u = torch.sign(self.beta1 * m + (1 - self.beta1) * gr)
                if g.weight_decay:
                    u = u + g.weight_decay * pv
                p.data.copy_((pv - g.lr * u).to(p.dtype))
                m.mul_(self.beta2).add_(gr, alpha=1 - self.beta2)


class LAMB(Optimizer):
    """Layer-wise adaptive moments: per-tensor trust ratio ||p|| / ||update||, eps 1e-6."""

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-6,
                 weight_decay: float = 0.0):
        super().__init__(as_groups(params, lr, weight_decay))
        self.beta1, self.beta2 = betas
        self.eps = eps
        self.t = 0

    def _begin_step(self):
        self.t += 1

    def _extra_scalars(self):
        return {"t": self.t}

    def _load_extra_scalars(self, d):
        self.t = int(d.get("t", 0))

    def _update(self, g: Group, params: List[torch.Tensor]):
        bc1 = 1 - self.beta1 ** self.t
        bc2 = 1 - self.beta2 ** self.t
        for ps in mt.by_dtype(params):
            ms = [self.state(p).buf("m", p, state_dtype(p)) for p in ps]
            vs = [self.state(p).buf("v", p, state_dtype(p)) for p in ps]
            if mt.native(ps[0]):
                masters = [self.master(p) for p in ps]
                grads = [p.grad for p in ps]
                norms = torch.zeros(2 * len(ps), dtype=torch.float32, device=ps[0].device)
                hy = [g.lr, g.weight_decay, self.beta1, self.beta2, self.eps, bc1, bc2, 0, 1.0]
                # phase 1 overwrites the gradients with the update direction
                mt.launch(mt.LAMB1, ps, grads, masters, ms, vs, hy, 0, norms, 2)
                mt.launch(mt.LAMB2, ps, grads, masters, ms, vs, hy, 0, norms, 2)
                continue
            for p, m, v in zip(ps, ms, vs):
                ct = state_dtype(p)
                gr, pv = p.grad.to(ct), p.data.to(ct)
                m.mul_(self.beta1).add_(gr, alpha=1 - self.beta1)
                v.mul_(self.beta2).addcmul_(gr, gr, value=1 - self.beta2)
                u = (m / bc1) / ((v / bc2).sqrt() + self.eps)
                if g.weight_decay:
                    u = u + g.weight_decay * pv
                pn, un = pv.norm().item(), u.norm().item()
                trust = pn / un if pn > 0 and un > 0 else 1.0
                p.data.copy_((pv - g.lr * trust * u).to(p.dtype))

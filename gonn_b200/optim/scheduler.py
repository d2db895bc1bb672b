"""Learning-rate schedulers (optim/scheduler.go:6-380).  Group aware: recursive schedules
multiply every group's current lr (``scale_lrs``), closed-form schedules set each group's lr
from the base lr captured at construction (``set_lrs``)."""
from __future__ import annotations

import math
from typing import Callable, Sequence


class Scheduler:
    def __init__(self, opt):
        self.opt = opt
        self.base_lrs = [g.lr for g in opt.Groups()]

    def scale_lrs(self, gamma: float):
        for g in self.opt.Groups():
            g.lr *= gamma

    def set_lrs(self, f: Callable[[float], float]):
        for g, b in zip(self.opt.Groups(), self.base_lrs):
            g.lr = f(b)

    def step(self):
        raise NotImplementedError

    def Step(self, *a):
        return self.step(*a)


class StepLR(Scheduler):
    def __init__(self, opt, step_size: int, gamma: float = 0.1):
        super().__init__(opt)
        self.step_size, self.gamma, self.count = step_size, gamma, 0

    def step(self):
        self.count += 1
        if self.step_size > 0 and self.count % self.step_size == 0:
            self.scale_lrs(self.gamma)


class MultiStepLR(Scheduler):
    def __init__(self, opt, milestones: Sequence[int], gamma: float = 0.1):
        super().__init__(opt)
        self.milestones, self.gamma, self.count = list(milestones), gamma, 0

    def step(self):
        self.count += 1
        if self.count in self.milestones:
            self.scale_lrs(self.gamma)


class ExponentialLR(Scheduler):
    def __init__(self, opt, gamma: float):
        super().__init__(opt)
        self.gamma = gamma

    def step(self):
        self.scale_lrs(self.gamma)


class CosineAnnealingLR(Scheduler):
    def __init__(self, opt, T_max: int, eta_min: float = 0.0):
        super().__init__(opt)
        self.T_max, self.eta_min, self.t = T_max, eta_min, 0

    def step(self):
        self.t += 1
        if self.T_max <= 0:
            return
        c = math.cos(math.pi * self.t / self.T_max)
        self.set_lrs(lambda b: self.eta_min + 0.5 * (b - self.eta_min) * (1 + c))


class LinearLR(Scheduler):
    def __init__(self, opt, start_factor: float = 1.0 / 3, end_factor: float = 1.0, total_iters: int = 5):
        super().__init__(opt)
        self.sf, self.ef, self.total, self.count = start_factor, end_factor, total_iters, 0
        self.set_lrs(lambda b: b * start_factor)      # the start factor applies immediately

    def step(self):
        self.count += 1
        f = self.ef
        if self.total > 0 and self.count < self.total:
            f = self.sf + (self.ef - self.sf) * self.count / self.total
        self.set_lrs(lambda b: b * f)


class ReduceLROnPlateau(Scheduler):
    """Metric scheduler: ``step(loss)``; scales by ``factor`` after more than ``patience`` calls
    without an improvement of at least ``threshold``."""

    def __init__(self, opt, factor: float = 0.1, threshold: float = 1e-4, patience: int = 10):
        super().__init__(opt)
        self.factor, self.threshold, self.patience = factor, threshold, patience
        self.best, self.bad = None, 0

    def step(self, loss_value: float):
        if self.best is None or loss_value < self.best - self.threshold:
            self.best, self.bad = loss_value, 0
            return
        self.bad += 1
        if self.bad > self.patience:
            self.scale_lrs(self.factor)
            self.bad = 0


class PolynomialLR(Scheduler):
    def __init__(self, opt, total_iters: int, power: float = 1.0):
        super().__init__(opt)
        self.total, self.power, self.count = total_iters, power, 0

    def step(self):
        self.count += 1
        if self.total <= 0:
            return
        if self.count >= self.total:
            self.set_lrs(lambda b: 0.0)
            return
        s = (1 - self.count / self.total) ** self.power
        self.set_lrs(lambda b: b * s)


class ChainedScheduler:
    def __init__(self, *schedulers):
        self.schedulers = list(schedulers)

    def step(self):
        for s in self.schedulers:
            s.step()

    Step = step


class SequentialLR:
    """Scheduler i is active while count <= milestones[i]; the last one afterwards."""

    def __init__(self, schedulers, milestones: Sequence[int]):
        self.schedulers, self.milestones, self.count = list(schedulers), list(milestones), 0

    def step(self):
        self.count += 1
        idx = 0
        for i, m in enumerate(self.milestones):
            if self.count > m:
                idx = i + 1
            else:
                break
        idx = min(idx, len(self.schedulers) - 1)
        if idx >= 0:
            self.schedulers[idx].step()

    Step = step


class CyclicLR(Scheduler):
    """Triangular cycle between base_lr and max_lr with half-period ``step_size``."""

    def __init__(self, opt, base_lr: float, max_lr: float, step_size: int):
        super().__init__(opt)
        self.base_lr, self.max_lr, self.step_size, self.count = base_lr, max_lr, step_size, 0
        self.set_lrs(lambda b: base_lr)

    def step(self):
        self.count += 1
        if self.step_size <= 0:
            return
        cycle = math.floor(1 + self.count / (2 * self.step_size))
        x = abs(self.count / self.step_size - 2 * cycle + 1)
        lr = self.base_lr + (self.max_lr - self.base_lr) * max(0.0, 1 - x)
        self.set_lrs(lambda b: lr)


class OneCycleLR(Scheduler):
    """Linear warm-up from the base lr to max_lr over the first half, linear decay back."""

    def __init__(self, opt, max_lr: float, total_steps: int):
        super().__init__(opt)
        self.max_lr, self.total, self.count = max_lr, total_steps, 0

    def step(self):
        self.count += 1
        if self.total <= 0:
            return
        half, t = self.total / 2, float(self.count)

        def f(b):
            if t <= half:
                return b + (self.max_lr - b) * t / half
            if t <= self.total:
                return self.max_lr + (b - self.max_lr) * (t - half) / half
            return b
        self.set_lrs(f)

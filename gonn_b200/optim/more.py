"""The remaining optimizers, as tensor-expression updates with the reference's exact rules
(optim/{rmsprop,adagrad,adadelta,nadam,adamax,radam,rprop,adafactor,asgd,sparse_adam,lbfgs}.go).
State buffer names are the frozen ones of optim/state.go:3-17.  Updates run in fp32 (fp64 for
fp64 parameters) on whatever device the parameter lives on.
"""
from __future__ import annotations

import math
from typing import Callable, List

import torch

from .base import Group, Optimizer, as_groups, state_dtype


def _wd(g, p, wd):
    return g + wd * p if wd else g


class _Simple(Optimizer):
    """Per-parameter update template: subclasses implement ``_one(group, p, data, grad, state)``
    where ``data`` is a working copy in the state dtype that is written back afterwards."""

    def _update(self, group: Group, params: List[torch.Tensor]):
        for p in params:
            ct = state_dtype(p)
            data = self.master(p) if p.dtype in (torch.bfloat16, torch.float16) else p.data
            if data.dtype != ct:
                data = data.to(ct)
            new = self._one(group, p, data, p.grad.to(ct), self.state(p))
            if new is not None:
                data = new
            if p.dtype in (torch.bfloat16, torch.float16):
                self.master(p).copy_(data)
            p.data.copy_(data.to(p.dtype))


class RMSprop(_Simple):
    def __init__(self, params, lr=0.01, alpha=0.99, eps=1e-8, momentum=0.0, weight_decay=0.0):
        super().__init__(as_groups(params, lr, weight_decay))
        self.alpha, self.eps, self.momentum = alpha, eps, momentum

    def _one(self, g, p, data, grad, st):
        grad = _wd(grad, data, g.weight_decay)
        sa = st.buf("square_avg", p, data.dtype)
        sa.mul_(self.alpha).addcmul_(grad, grad, value=1 - self.alpha)
        denom = sa.sqrt() + self.eps
        if self.momentum:
            mb = st.buf("momentum_buf", p, data.dtype)
            mb.mul_(self.momentum).add_(grad / denom)
            return data - g.lr * mb
        return data - g.lr * grad / denom


class Adagrad(_Simple):
    def __init__(self, params, lr=0.01, lr_decay=0.0, eps=1e-10, weight_decay=0.0):
        super().__init__(as_groups(params, lr, weight_decay))
        self.lr_decay, self.eps, self.t = lr_decay, eps, 0

    def _begin_step(self):
        self.t += 1

    def _one(self, g, p, data, grad, st):
        grad = _wd(grad, data, g.weight_decay)
        clr = g.lr / (1 + (self.t - 1) * self.lr_decay)
        s = st.buf("sum", p, data.dtype)
        s.addcmul_(grad, grad)
        return data - clr * grad / (s.sqrt() + self.eps)


class Adadelta(_Simple):
    def __init__(self, params, lr=1.0, rho=0.9, eps=1e-6, weight_decay=0.0):
        super().__init__(as_groups(params, lr, weight_decay))
        self.rho, self.eps = rho, eps

    def _one(self, g, p, data, grad, st):
        grad = _wd(grad, data, g.weight_decay)
        sa, ad = st.buf("square_avg", p, data.dtype), st.buf("acc_delta", p, data.dtype)
        sa.mul_(self.rho).addcmul_(grad, grad, value=1 - self.rho)
        delta = (ad + self.eps).sqrt() / (sa + self.eps).sqrt() * grad
        ad.mul_(self.rho).addcmul_(delta, delta, value=1 - self.rho)
        return data - g.lr * delta


class NAdam(_Simple):
    def __init__(self, params, lr=2e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, momentum_decay=4e-3):
        super().__init__(as_groups(params, lr, weight_decay))
        self.beta1, self.beta2 = betas
        self.eps, self.momentum_decay = eps, momentum_decay
        self.t, self.mu_product = 0, 1.0

    def _begin_step(self):
        self.t += 1
        t = float(self.t)
        self._mu_t = self.beta1 * (1 - 0.5 * 0.96 ** (t * self.momentum_decay))
        self._mu_next = self.beta1 * (1 - 0.5 * 0.96 ** ((t + 1) * self.momentum_decay))
        self.mu_product *= self._mu_t
        self._mu_prod_next = self.mu_product * self._mu_next
        self._bc2 = 1 - self.beta2 ** t

    def _extra_scalars(self):
        return {"t": self.t, "mu_product": self.mu_product}

    def _load_extra_scalars(self, d):
        self.t, self.mu_product = int(d.get("t", 0)), float(d.get("mu_product", 1.0))

    def _one(self, g, p, data, grad, st):
        grad = _wd(grad, data, g.weight_decay)
        m, v = st.buf("m", p, data.dtype), st.buf("v", p, data.dtype)
        m.mul_(self.beta1).add_(grad, alpha=1 - self.beta1)
        v.mul_(self.beta2).addcmul_(grad, grad, value=1 - self.beta2)
        m_hat = self._mu_next * m / (1 - self._mu_prod_next) + (1 - self._mu_t) * grad / (1 - self.mu_product)
        return data - g.lr * m_hat / ((v / self._bc2).sqrt() + self.eps)


class Adamax(_Simple):
    def __init__(self, params, lr=2e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0):
        super().__init__(as_groups(params, lr, weight_decay))
        self.beta1, self.beta2 = betas
        self.eps, self.t = eps, 0

    def _begin_step(self):
        self.t += 1

    def _one(self, g, p, data, grad, st):
        grad = _wd(grad, data, g.weight_decay)
        m, u = st.buf("m", p, data.dtype), st.buf("u", p, data.dtype)
        m.mul_(self.beta1).add_(grad, alpha=1 - self.beta1)
        torch.maximum(u * self.beta2, grad.abs(), out=u)
        return data - (g.lr / (1 - self.beta1 ** self.t)) * m / (u + self.eps)


class RAdam(_Simple):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0):
        super().__init__(as_groups(params, lr, weight_decay))
        self.beta1, self.beta2 = betas
        self.eps, self.t = eps, 0

    def _begin_step(self):
        self.t += 1
        t = float(self.t)
        self._bc1, self._bc2 = 1 - self.beta1 ** t, 1 - self.beta2 ** t
        rho_inf = 2 / (1 - self.beta2) - 1
        rho_t = rho_inf - 2 * t * self.beta2 ** t / self._bc2
        self._rect = math.sqrt(((rho_t - 4) * (rho_t - 2) * rho_inf) / ((rho_inf - 4) * (rho_inf - 2) * rho_t)) \
            if rho_t > 4 else None

    def _one(self, g, p, data, grad, st):
        grad = _wd(grad, data, g.weight_decay)
        m, v = st.buf("m", p, data.dtype), st.buf("v", p, data.dtype)
        m.mul_(self.beta1).add_(grad, alpha=1 - self.beta1)
        v.mul_(self.beta2).addcmul_(grad, grad, value=1 - self.beta2)
        m_hat = m / self._bc1
        if self._rect is not None:
            return data - g.lr * self._rect * m_hat / ((v / self._bc2).sqrt() + self.eps)
        return data - g.lr * m_hat


class Rprop(_Simple):
    def __init__(self, params, lr=0.01, etas=(0.5, 1.2), step_sizes=(1e-6, 50.0)):
        super().__init__(as_groups(params, lr))
        self.eta_minus, self.eta_plus = etas
        self.step_min, self.step_max = step_sizes

    def _one(self, g, p, data, grad, st):
        prev = st.buf("prev_grad", p, data.dtype)
        step = st.buf_fill("step_size", p, g.lr, data.dtype)
        sp = prev * grad
        step.copy_(torch.where(sp > 0, (step * self.eta_plus).clamp(max=self.step_max),
                               torch.where(sp < 0, (step * self.eta_minus).clamp(min=self.step_min), step)))
        geff = torch.where(sp < 0, torch.zeros_like(grad), grad)
        new = data - torch.sign(geff) * step
        prev.copy_(torch.where(sp < 0, torch.zeros_like(grad), torch.sign(geff) * grad.abs()))
        return new


class Adafactor(_Simple):
    """Non-factored Adafactor: relative step min(1/sqrt(t), lr), update clipping by RMS."""

    def __init__(self, params, lr=1e-2, eps=(1e-30, 1e-3), clip_threshold=1.0, decay_rate=-0.8):
        super().__init__(as_groups(params, lr))
        self.eps1, self.eps2 = eps
        self.clip_threshold, self.decay_rate = clip_threshold, decay_rate

    def _one(self, g, p, data, grad, st):
        v = st.buf("v", p, data.dtype)
        t = st.scalar("step") + 1
        st.set_scalar("step", t)
        beta2hat = 1 - t ** self.decay_rate
        rel = min(1 / math.sqrt(t), g.lr)
        rms = lambda x: float(x.pow(2).mean().sqrt()) if x.numel() else 0.0
        alpha = max(self.eps2, rms(data)) * rel
        v.mul_(beta2hat).add_((grad * grad + self.eps1) * (1 - beta2hat))
        upd = grad / v.sqrt()
        denom = max(1.0, rms(upd) / self.clip_threshold)
        return data - alpha * upd / denom


class ASGD(_Simple):
    """Averaged SGD; ``AveragedParam(p)`` returns the running average ``ax``."""

    def __init__(self, params, lr=0.01, lambd=1e-4, alpha=0.75, t0=1e6, weight_decay=0.0):
        super().__init__(as_groups(params, lr, weight_decay))
        self.lambd, self.alpha, self.t0 = lambd, alpha, t0

    def _one(self, g, p, data, grad, st):
        if not st.has("ax"):
            st.set_scalar("eta", g.lr); st.set_scalar("mu", 1); st.set_scalar("step", 0)
        ax = st.buf("ax", p, data.dtype)
        st.set_scalar("step", st.scalar("step") + 1)
        t, eta, mu = st.scalar("step"), st.scalar("eta"), st.scalar("mu")
        grad = _wd(grad, data, g.weight_decay)
        new = data * (1 - self.lambd * eta) - eta * grad
        if mu != 1:
            ax.add_(mu * (new - ax))
        else:
            ax.copy_(new)
        st.set_scalar("eta", g.lr / (1 + self.lambd * g.lr * t) ** self.alpha)
        st.set_scalar("mu", 1 / max(1.0, t - self.t0))
        return new

    def AveragedParam(self, p):
        return self.state(p).bufs.get("ax")


class SparseAdam(_Simple):
    """Adam that only touches entries with a non-zero gradient; per-element step counts
    (dense emulation, like the reference)."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8):
        super().__init__(as_groups(params, lr))
        self.beta1, self.beta2 = betas
        self.eps = eps

    def _one(self, g, p, data, grad, st):
        m, v, cnt = st.buf("m", p, data.dtype), st.buf("v", p, data.dtype), st.buf("step", p, data.dtype)
        nz = grad != 0
        cnt.add_(nz.to(cnt.dtype))
        t = cnt.clamp_min(1)
        m_new = self.beta1 * m + (1 - self.beta1) * grad
        v_new = self.beta2 * v + (1 - self.beta2) * grad * grad
        m.copy_(torch.where(nz, m_new, m))
        v.copy_(torch.where(nz, v_new, v))
        upd = g.lr * (m / (1 - self.beta1 ** t)) / ((v / (1 - self.beta2 ** t)).sqrt() + self.eps)
        return torch.where(nz, data - upd, data)


class LBFGS:
    """Limited-memory BFGS with a closure: two-loop recursion, Armijo backtracking, history 10,
    max_iter 20 (optim/lbfgs.go:15-286).  ``step(closure)`` re-evaluates the loss as needed;
    it is not an ``Optimizer.step``."""

    def __init__(self, params, lr=1.0, max_iter=20, history_size=10, tolerance_grad=1e-7,
                 tolerance_change=1e-9, c1=1e-4):
        self.params = [p for p in params]
        self.lr, self.max_iter, self.history = lr, max_iter, history_size
        self.tol_g, self.tol_c, self.c1 = tolerance_grad, tolerance_change, c1
        self.s: List[torch.Tensor] = []
        self.y: List[torch.Tensor] = []

    # exported fields of the reference's struct (optim/lbfgs.go:15-30)
    HistorySize = property(lambda self: self.history, lambda self, v: setattr(self, "history", int(v)))
    MaxIter = property(lambda self: self.max_iter, lambda self, v: setattr(self, "max_iter", int(v)))

    def parameters(self):
        return self.params

    def zero_grad(self):
        for p in self.params:
            p.grad = None

    def _flat(self, what):
        return torch.cat([(getattr(p, what) if what == "data" else
                           (p.grad if p.grad is not None else torch.zeros_like(p))).reshape(-1).double()
                          for p in self.params])

    def _set(self, flat):
        off = 0
        with torch.no_grad():
            for p in self.params:
                n = p.numel()
                p.copy_(flat[off:off + n].reshape(p.shape).to(p.dtype))
                off += n

    def step(self, closure: Callable[[], float]) -> float:
        def evaluate():
            self.zero_grad()
            with torch.enable_grad():
                l = closure()
            return float(l.detach()) if hasattr(l, "detach") else float(l)
        loss = evaluate()
        g = self._flat("grad")
        for _ in range(self.max_iter):
            if g.abs().max() <= self.tol_g:
                break
            q = g.clone()
            alphas = []
            for s, y in zip(reversed(self.s), reversed(self.y)):
                rho = 1.0 / (y @ s)
                a = rho * (s @ q)
                alphas.append((a, rho, s, y))
                q -= a * y
            if self.s:
                q *= (self.s[-1] @ self.y[-1]) / (self.y[-1] @ self.y[-1])
            for a, rho, s, y in reversed(alphas):
                q += (a - rho * (y @ q)) * s
            d = -q
            gd = float(g @ d)
            if gd >= 0:
                d, gd = -g, -float(g @ g)
            x0 = self._flat("data")
            t = self.lr
            ok = False
            for _ls in range(25):
                self._set(x0 + t * d)
                new_loss = evaluate()
                if new_loss <= loss + self.c1 * t * gd:
                    ok = True
                    break
                t *= 0.5
            if not ok:
                self._set(x0)
                evaluate()
                break
            g_new = self._flat("grad")
            s, y = t * d, g_new - g
            if float(y @ s) > 1e-10:
                self.s.append(s); self.y.append(y)
                if len(self.s) > self.history:
                    self.s.pop(0); self.y.pop(0)
            change = abs(new_loss - loss)
            loss, g = new_loss, g_new
            if change < self.tol_c:
                break
        return loss

    Step = step

"""Functional calls with replaced parameters (nn/stateless.go:59-257)."""
from __future__ import annotations

import contextlib
from typing import Callable, Dict, Sequence

import torch


@contextlib.contextmanager
def WithReplacedParams(module: torch.nn.Module, replace: Dict[str, torch.Tensor]):
    """Temporarily swaps parameter / buffer *values* by dotted name; restored on exit even if
    the body raises (the reference swaps Data in place and restores in a defer)."""
    named = dict(module.named_parameters())
    named.update(dict(module.named_buffers()))
    unknown = [k for k in replace if k not in named]
    if unknown:
        raise KeyError(f"WithReplacedParams: unknown names {unknown}")
    saved = {}
    try:
        for k, v in replace.items():
            t = named[k]
            if tuple(v.shape) != tuple(t.shape):
                raise ValueError(f"WithReplacedParams: shape mismatch for {k}")
            saved[k] = t.data
            t.data = v.detach().to(dtype=t.dtype, device=t.device)
        yield module
    finally:
        for k, d in saved.items():
            named[k].data = d


def FunctionalCall(module: torch.nn.Module, x, replace: Dict[str, torch.Tensor]):
    """``module(x)`` evaluated with the given tensors in place of the named parameters; the
    result is differentiable with respect to the replacements."""
    return torch.func.functional_call(module, dict(replace), (x,) if not isinstance(x, tuple) else x)


def FunctionalCallMulti(module: torch.nn.Module, replace: Dict[str, torch.Tensor], *inputs):
    return torch.func.functional_call(module, dict(replace), inputs)


def WithGradsToReplacements():
    """Option for ``FunctionalCallGrad`` / ``FunctionalCallGradMulti``: besides returning the
    gradients by name, accumulate each one into the ``.grad`` of the tensor that replaced the
    parameter (allocated when missing), the way ``torch.func.functional_call`` users expect
    (nn/stateless.go:144-152).  The module's own parameters keep their ``.grad`` untouched."""
    return "grads_to_replacements"


def _harvest(rep, replace, loss, opts):
    grads = torch.autograd.grad(loss, list(rep.values()), allow_unused=True)
    out = {k: g for k, g in zip(rep, grads) if g is not None}
    if "grads_to_replacements" in opts:
        for k, g in out.items():
            t = replace[k]
            t.grad = g.detach().clone() if t.grad is None else t.grad + g.detach()
    return out


def FunctionalCallGrad(module: torch.nn.Module, x, replace: Dict[str, torch.Tensor],
                       loss_fn: Callable[[torch.Tensor], torch.Tensor], *opts):
    """Returns (loss, {name: dloss/dreplacement}); parameters that received no gradient are
    omitted (nn/stateless.go:214-231)."""
    rep = {k: v.detach().clone().requires_grad_(True) for k, v in replace.items()}
    loss = loss_fn(FunctionalCall(module, x, rep))
    return loss.detach(), _harvest(rep, replace, loss, opts)


def FunctionalCallGradMulti(module, replace, loss_fn, *inputs, opts=()):
    rep = {k: v.detach().clone().requires_grad_(True) for k, v in replace.items()}
    loss = loss_fn(FunctionalCallMulti(module, rep, *inputs))
    return loss.detach(), _harvest(rep, replace, loss, tuple(opts))

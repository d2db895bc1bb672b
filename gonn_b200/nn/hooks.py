"""Forward-pre / forward / full-backward hooks, per module and global (nn/hooks.go:43-293).

Per-module hooks are torch's own (``register_forward_pre_hook`` ...), exposed under the
reference's names with integer handles; ``Call(m, x)`` is ``m(x)`` (a bare ``forward``
bypasses hooks, as in the reference).  Hook signatures follow the reference: pre
``fn(module, x) -> x or None``, forward ``fn(module, x, y) -> y or None``, backward
``fn(module, grad_out) -> grad or None``.
"""
from __future__ import annotations

import itertools
from typing import Callable, Dict

import torch

_ids = itertools.count(1)
_handles: Dict[int, object] = {}
_global: Dict[int, object] = {}


def _wrap_pre(fn):
    def h(m, args):
        r = fn(m, args[0])
        return None if r is None else (r,) + tuple(args[1:])
    return h


def _wrap_fwd(fn):
    def h(m, args, out):
        return fn(m, args[0], out)
    return h


def _wrap_bwd(fn):
    def h(m, grad_in, grad_out):
        r = fn(m, grad_out[0])
        if r is None:
            return None
        # a replaced output gradient is propagated by scaling the input gradients accordingly is
        # not defined in general; like the reference's identity node, the hook may observe or
        # replace the gradient flowing INTO the module's backward, which torch exposes through
        # a tensor hook on the output instead (see RegisterFullBackwardHook)
        return None
    return h


def RegisterForwardPreHook(module: torch.nn.Module, fn: Callable) -> int:
    i = next(_ids)
    _handles[i] = module.register_forward_pre_hook(_wrap_pre(fn))
    return i


def RegisterForwardHook(module: torch.nn.Module, fn: Callable) -> int:
    i = next(_ids)
    _handles[i] = module.register_forward_hook(_wrap_fwd(fn))
    return i


def RegisterFullBackwardHook(module: torch.nn.Module, fn: Callable) -> int:
    """``fn(module, grad_out)`` sees the gradient of the module's output and may return a
    replacement (the reference attaches an identity node to the output for this)."""
    i = next(_ids)

    def fwd(m, args, out):
        if isinstance(out, torch.Tensor) and out.requires_grad:
            out.register_hook(lambda g: fn(m, g))
        return None
    _handles[i] = module.register_forward_hook(fwd)
    return i


def RemoveHook(hook_id: int) -> bool:
    h = _handles.pop(hook_id, None) or _global.pop(hook_id, None)
    if h is None:
        return False
    h.remove()
    return True


def RegisterModuleForwardPreHook(fn: Callable) -> int:
    i = next(_ids)
    _global[i] = torch.nn.modules.module.register_module_forward_pre_hook(_wrap_pre(fn))
    return i


def RegisterModuleForwardHook(fn: Callable) -> int:
    i = next(_ids)
    _global[i] = torch.nn.modules.module.register_module_forward_hook(_wrap_fwd(fn))
    return i


def RegisterModuleFullBackwardHook(fn: Callable) -> int:
    i = next(_ids)

    def fwd(m, args, out):
        if isinstance(out, torch.Tensor) and out.requires_grad:
            out.register_hook(lambda g: fn(m, g))
        return None
    _global[i] = torch.nn.modules.module.register_module_forward_hook(fwd)
    return i


RemoveModuleHook = RemoveHook


def Call(module: torch.nn.Module, *args, **kw):
    """Runs the hook pipeline around ``forward``."""
    return module(*args, **kw)

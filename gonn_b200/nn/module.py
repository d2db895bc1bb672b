"""Module system: registration-ordered parameters with dotted names, buffers,
train/eval flag, containers.

``Module`` is ``torch.nn.Module`` plus the reference's vocabulary
(nn/module.go:12-209): ``Parameters()`` / ``NamedParameters()`` / ``Buffers()``
/ ``SetTraining()`` aliases, ``FilterParams`` for building optimizer groups by
name, ``Sequential`` whose children are named "0", "1", ...  Parameter order is
the module's own parameters in registration order, then children depth-first —
the same order torch uses, so state-dict keys match the reference's naming
contract.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Callable, Dict, Iterable, List, Tuple

import torch
from torch import nn as _tnn


def _pad_side(dim_from_last: int, side: int):
    return lambda m: m.pads[len(m.pads) - 1 - dim_from_last][side]


# exported field names of the reference's module structs that differ from the attribute here by more
# than spelling: name -> attribute names (or getters) tried in order
_FIELD_NAMES = {
    "Kernel": ("kernel_size", "k"), "Pad": ("padding", "p"), "Stride": ("s",), "Dilation": ("d",),
    "In1Features": ("in1",), "In2Features": ("in2",), "Dropouts": ("dropout",), "Axis": ("dim",),
    "EmbDim": ("embed_dim", lambda m: m.attn.embed_dim), "EmbedDim": (lambda m: m.encoder.layers[0].attn.embed_dim,),
    "NumHeads": (lambda m: m.attn.num_heads, lambda m: m.encoder.layers[0].attn.num_heads),
    "DimFF": (lambda m: m.ff1.out_features, lambda m: m.linear1.out_features),
    "NumParams": (lambda m: m.weight.numel(),), "ScaleFactor": ("scale",), "UpscaleFactor": ("r",),
    "DownscaleFactor": ("r",), "G": ("weight_g",), "V": ("weight_v",), "Weight": ("weight_orig",),
    "InFeatures": (lambda m: m.EffectiveWeight().shape[1],), "OutFeatures": (lambda m: m.EffectiveWeight().shape[0],),
    "ShortlistSize": ("shortlist",), "HeadSize": (lambda m: m.shortlist + m.n_clusters,),
    "HeadBias": (lambda m: m.head.bias is not None,),
    "OutSize": (lambda m: m.output_size[0],), "OutD": (lambda m: m.output_size[-3],),
    "OutH": (lambda m: m.output_size[-2],), "OutW": (lambda m: m.output_size[-1],),
    "Left": (_pad_side(0, 0),), "Right": (_pad_side(0, 1),), "Top": (_pad_side(1, 0),), "Bottom": (_pad_side(1, 1),),
    "Front": (_pad_side(2, 0),), "Back": (_pad_side(2, 1),),
}


class Module(_tnn.Module):
    """Base class of every layer."""

    # ---- reference-style field names ---------------------------------------------------
    def __getattr__(self, name: str):
        """Exported field names of the reference resolve to the attribute of this module:
        ``lin.Weight`` is ``lin.weight``, ``lin.InFeatures`` is ``lin.in_features``,
        ``bn.RunningMean`` is ``bn.running_mean``.  The alternative spellings are tried only after
        torch's own lookup of parameters / buffers / children has failed; the usual lookups pay
        one extra Python call."""
        try:
            return super().__getattr__(name)
        except AttributeError:
            if name[:1].isupper():
                snake = "".join("_" + c.lower() if c.isupper() and i else c.lower() for i, c in enumerate(name))
                for alt in (snake, name.lower()) + _FIELD_NAMES.get(name, ()):
                    if alt != name:
                        try:
                            return alt(self) if callable(alt) else getattr(self, alt)
                        except (AttributeError, IndexError, TypeError):
                            pass
            raise

    # ---- reference-style accessors -------------------------------------------------
    def Parameters(self) -> List[torch.nn.Parameter]:
        return list(self.parameters())

    def NamedParameters(self) -> List[Tuple[str, torch.nn.Parameter]]:
        return list(self.named_parameters())

    def Buffers(self) -> List[Tuple[str, torch.Tensor]]:
        return list(self.named_buffers())

    # ---- hooks as methods (nn/hooks.go:86-160); the functions of the same names take the module
    def RegisterForwardPreHook(self, fn) -> int:
        from . import hooks
        return hooks.RegisterForwardPreHook(self, fn)

    def RegisterForwardHook(self, fn) -> int:
        from . import hooks
        return hooks.RegisterForwardHook(self, fn)

    def RegisterFullBackwardHook(self, fn) -> int:
        from . import hooks
        return hooks.RegisterFullBackwardHook(self, fn)

    def RemoveHook(self, hook_id: int) -> bool:
        from . import hooks
        return hooks.RemoveHook(hook_id)

    def Forward(self, *args, **kwargs):
        """The reference's spelling of the forward pass (nn/module.go:29-33).  As there, it runs
        the layer directly; hooks run when the module is called (``m(x)`` or ``nn.Call(m, x)``)."""
        return self.forward(*args, **kwargs)

    def SetTraining(self, flag: bool) -> "Module":
        return self.train(flag)

    def Train(self) -> "Module":
        return self.train(True)

    def Eval(self) -> "Module":
        return self.train(False)

    @property
    def Training(self) -> bool:
        return self.training

    # ---- registration helpers (reference: Base.reg / regBuf / regChild) --------------
    def reg(self, name: str, tensor: torch.Tensor) -> torch.nn.Parameter:
        p = tensor if isinstance(tensor, torch.nn.Parameter) else torch.nn.Parameter(tensor)
        self.register_parameter(name, p)
        return p

    RegisterParam = reg

    def reg_buf(self, name: str, tensor: torch.Tensor) -> torch.Tensor:
        self.register_buffer(name, tensor)
        return tensor

    RegisterBuffer = reg_buf

    def reg_child(self, name: str, child: _tnn.Module) -> _tnn.Module:
        self.add_module(name, child)
        return child

    RegisterChild = reg_child

    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters())


def FilterParams(module: _tnn.Module, pred: Callable[..., bool]):
    """Parameters selected by ``pred``, which takes the dotted name as in the reference
    (nn/module.go:167-175) or the name and the tensor."""
    import inspect
    try:
        two = len(inspect.signature(pred).parameters) >= 2
    except (TypeError, ValueError):
        two = False
    return [p for n, p in module.named_parameters() if (pred(n, p) if two else pred(n))]


def NamedParameters(module: _tnn.Module):
    """``[Param(name, tensor), ...]`` in registration order (nn/module.go:12-15, 120-135)."""
    from .types import Param
    return [Param(n, p) for n, p in module.named_parameters()]


filter_params = FilterParams


class Sequential(Module):
    """Runs children in order; children are named "0", "1", ... (nn/module.go:178-209).
    Children are invoked through ``__call__`` so hooks fire, like the reference's ``Call``."""

    def __init__(self, *layers: _tnn.Module):
        super().__init__()
        for l in layers:
            self.Add(l)

    def Add(self, layer: _tnn.Module) -> "Sequential":
        self.add_module(str(len(self._modules)), layer)
        return self

    add = Add

    def __len__(self):
        return len(self._modules)

    Len = __len__

    def __getitem__(self, i):
        if isinstance(i, slice):
            return Sequential(*list(self._modules.values())[i])
        return list(self._modules.values())[i]

    def __iter__(self):
        return iter(self._modules.values())

    def forward(self, x):
        for m in self._modules.values():
            x = m(x)
        return x


class ModuleList(_tnn.ModuleList, Module):
    """Indexable list of children named by position (nn/containers.go:27-80)."""

    def Append(self, m):
        self.append(m)
        return self

    def Len(self):
        return len(self)

    def Get(self, i: int):
        return self[i]


class ModuleDict(Module):
    """Children keyed by name, iterated in sorted key order (nn/containers.go:82-140)."""

    def __init__(self, modules: Dict[str, _tnn.Module] = None):
        super().__init__()
        for k in sorted(modules or {}):
            self.add_module(k, modules[k])

    def Set(self, key: str, m: _tnn.Module):
        self._modules[key] = m
        self._modules = OrderedDict(sorted(self._modules.items()))
        return self

    __setitem__ = Set

    def Get(self, key: str):
        return self._modules[key]

    __getitem__ = Get

    def Keys(self):
        return list(self._modules.keys())

    keys = Keys

    def __len__(self):
        return len(self._modules)

    Len = __len__

    def __contains__(self, k):
        return k in self._modules

    def items(self):
        return self._modules.items()

    def values(self):
        return self._modules.values()


class ParameterList(_tnn.ParameterList, Module):
    """Parameters named "0", "1", ... (nn/containers.go:142-185)."""

    def Append(self, p):
        self.append(p if isinstance(p, torch.nn.Parameter) else torch.nn.Parameter(p))
        return self

    def Get(self, i: int):
        return self[i]

    def Len(self):
        return len(self)


class ParameterDict(Module):
    """Parameters keyed by name, sorted key order (nn/containers.go:187-229)."""

    def __init__(self, params: Dict[str, torch.Tensor] = None):
        super().__init__()
        for k in sorted(params or {}):
            self.Set(k, params[k])

    def Set(self, key: str, p: torch.Tensor):
        p = p if isinstance(p, torch.nn.Parameter) else torch.nn.Parameter(p)
        self._parameters[key] = p
        self._parameters = OrderedDict(sorted(self._parameters.items()))
        return self

    __setitem__ = Set

    def Get(self, key: str):
        return self._parameters[key]

    __getitem__ = Get

    def Keys(self):
        return list(self._parameters.keys())

    def __len__(self):
        return len(self._parameters)

    Len = __len__


class Identity(Module):
    def forward(self, x):
        return x


class Flatten(Module):
    """Flattens dims [start, end] (default: everything but the batch dim)."""

    def __init__(self, start_dim: int = 1, end_dim: int = -1):
        super().__init__()
        self.start_dim, self.end_dim = start_dim, end_dim

    def forward(self, x):
        return x.flatten(self.start_dim, self.end_dim)


class Unflatten(Module):
    def __init__(self, dim: int, sizes: Iterable[int]):
        super().__init__()
        self.dim, self.sizes = dim, tuple(sizes)

    def forward(self, x):
        return x.unflatten(self.dim, self.sizes)

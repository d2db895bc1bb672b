"""Optimizer base: parameter groups, named per-parameter state, the step template.

Mirrors optim/optimizer.go:15-24, optim/base.go:9-99, optim/group.go:20-24 and
optim/state.go:3-75: a ``Group`` holds literal ``lr`` / ``weight_decay`` values
(no inherit sentinel), state buffers have frozen names (``m``, ``v``,
``momentum_buf``, ...), parameters without a gradient are skipped, ``set_lr``
sets every group.

Mixed precision: a bf16/fp16 parameter gets an fp32 ``master`` buffer in its state
the first time it is stepped; the kernels update the master and write the rounded
value back to the parameter.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Optional, Sequence

import torch


@dataclass
class Group:
    """A parameter group (the analogue of a torch param_group)."""
    params: List[torch.Tensor]
    lr: float = 0.0
    weight_decay: float = 0.0

    # reference-style aliases
    @property
    def Params(self):
        return self.params

    @property
    def LR(self):
        return self.lr

    @LR.setter
    def LR(self, v):
        self.lr = v

    @property
    def WeightDecay(self):
        return self.weight_decay


class State:
    """Named buffers and scalars of one parameter, created lazily."""

    def __init__(self):
        self.bufs: Dict[str, torch.Tensor] = {}
        self.scalars: Dict[str, float] = {}

    def buf(self, name: str, like: torch.Tensor, dtype=None, fill: float = 0.0) -> torch.Tensor:
        b = self.bufs.get(name)
        if b is None:
            b = torch.full(like.shape, fill, dtype=dtype or like.dtype, device=like.device)
            self.bufs[name] = b
        return b

    Buf = buf

    def buf_fill(self, name, like, fill, dtype=None):
        return self.buf(name, like, dtype, fill)

    BufFill = buf_fill

    def has(self, name: str) -> bool:
        return name in self.bufs

    Has = has

    def scalar(self, name: str) -> float:
        return self.scalars.get(name, 0.0)

    Scalar = scalar

    def set_scalar(self, name: str, v: float) -> None:
        self.scalars[name] = float(v)

    SetScalar = set_scalar


def state_dtype(p: torch.Tensor) -> torch.dtype:
    return torch.float64 if p.dtype == torch.float64 else torch.float32


class Optimizer:
    """Base class; subclasses implement ``_update(group, params_with_grad)``."""

    def __init__(self, groups: Sequence[Group]):
        self.groups: List[Group] = [Group(list(g.params), g.lr, g.weight_decay) for g in groups]
        self.states: Dict[int, State] = {}
        self._base_lrs = [g.lr for g in self.groups]

    # ---- reference interface ----------------------------------------------------------
    def step(self, closure: Optional[Callable] = None):
        loss = closure() if closure is not None else None
        self._begin_step()
        for g in self.groups:
            ps = [p for p in g.params if p.grad is not None]
            if ps:
                self._update(g, ps)
        return loss

    Step = step

    def zero_grad(self, set_to_none: bool = False):
        for g in self.groups:
            for p in g.params:
                if p.grad is not None:
                    if set_to_none:
                        p.grad = None
                    else:
                        p.grad.zero_()

    ZeroGrad = zero_grad

    def parameters(self) -> List[torch.Tensor]:
        return [p for g in self.groups for p in g.params]

    Parameters = parameters

    def Groups(self) -> List[Group]:
        return self.groups

    @property
    def param_groups(self):
        return self.groups

    def lr(self) -> float:
        return self.groups[0].lr if self.groups else 0.0

    LR = lr

    def set_lr(self, lr: float) -> None:
        for g in self.groups:
            g.lr = lr

    SetLR = set_lr

    # ---- helpers ----------------------------------------------------------------------
    def state(self, p: torch.Tensor) -> State:
        s = self.states.get(id(p))
        if s is None:
            s = State()
            self.states[id(p)] = s
        return s

    def master(self, p: torch.Tensor) -> Optional[torch.Tensor]:
        """fp32 master copy for 16-bit parameters (None for fp32 / fp64)."""
        if p.dtype not in (torch.bfloat16, torch.float16):
            return None
        st = self.state(p)
        m = st.bufs.get("master")
        if m is None:
            m = p.detach().to(torch.float32).clone()
            st.bufs["master"] = m
        return m

    def _begin_step(self):
        pass

    def _update(self, group: Group, params: List[torch.Tensor]):
        raise NotImplementedError

    # ---- serialisable state -------------------------------------------------------------
    def state_dict(self, names: Optional[Dict[int, str]] = None) -> dict:
        """State keyed by parameter name (``names``: id(param) -> dotted name) or by position."""
        out = {"groups": [{"lr": g.lr, "weight_decay": g.weight_decay, "n": len(g.params)} for g in self.groups],
               "scalars": self._extra_scalars(), "state": {}}
        for gi, g in enumerate(self.groups):
            for pi, p in enumerate(g.params):
                st = self.states.get(id(p))
                if st is None:
                    continue
                key = names[id(p)] if names and id(p) in names else f"{gi}.{pi}"
                out["state"][key] = {"bufs": {k: v.detach().clone() for k, v in st.bufs.items()},
                                     "scalars": dict(st.scalars)}
        return out

    def load_state_dict(self, sd: dict, names: Optional[Dict[int, str]] = None) -> None:
        for g, gs in zip(self.groups, sd.get("groups", [])):
            g.lr, g.weight_decay = gs["lr"], gs["weight_decay"]
        self._load_extra_scalars(sd.get("scalars", {}))
        for gi, g in enumerate(self.groups):
            for pi, p in enumerate(g.params):
                key = names[id(p)] if names and id(p) in names else f"{gi}.{pi}"
                if key in sd["state"]:
                    st = self.state(p)
                    for k, v in sd["state"][key]["bufs"].items():
                        st.bufs[k] = v.to(device=p.device).clone()
                    st.scalars = dict(sd["state"][key]["scalars"])

    def _extra_scalars(self) -> dict:
        return {}

    def _load_extra_scalars(self, d: dict) -> None:
        pass


def as_groups(params_or_groups, lr: float, weight_decay: float = 0.0) -> List[Group]:
    """A flat parameter list becomes one group with the given defaults; a list of
    ``Group`` is used as is (defaults are NOT injected, like the reference's NewXGroups)."""
    items = list(params_or_groups)
    if items and isinstance(items[0], Group):
        return items
    if items and isinstance(items[0], dict):
        return [Group(list(d["params"]), d.get("lr", lr), d.get("weight_decay", weight_decay)) for d in items]
    return [Group(items, lr, weight_decay)]

"""Names of the reference's small types, for code that spells them out.

Go needs a named type for every callback signature, option bag and interface; Python does
not, so most of these are aliases or light records.  They exist so that a program written
against the reference's vocabulary (``nn.Param``, ``nn.LSTMState``, ``nn.ReduceSum``,
``nn.Child`` in a type annotation, ...) reads the same here.
"""
from __future__ import annotations

import enum
from typing import Callable, NamedTuple, Optional, Protocol, runtime_checkable

import torch

from .module import Module


class Param(NamedTuple):
    """A named parameter or buffer (nn/module.go:12-15)."""
    Name: str
    T: torch.Tensor


class LSTMState(NamedTuple):
    """Hidden and cell state of an LSTM step (nn/rnn.go:171-174); unpacks as ``h, c``."""
    H: torch.Tensor
    C: torch.Tensor


class Reduction(str, enum.Enum):
    """Loss reduction (nn/loss.go:16-25).  The members compare equal to the strings the
    loss functions take, so ``reduction=nn.ReduceSum`` and ``reduction="sum"`` are the same."""
    ReduceMean = "mean"
    ReduceSum = "sum"
    ReduceNone = "none"


ReduceMean, ReduceSum, ReduceNone = Reduction.ReduceMean, Reduction.ReduceSum, Reduction.ReduceNone

# every module carries its own parameter / buffer / mode state (the reference's embedded Base);
# Child is the part of that surface multi-input modules share (nn/module.go:21-26, 54-63)
Base = Module


@runtime_checkable
class Child(Protocol):
    def Parameters(self): ...
    def NamedParameters(self): ...
    def Buffers(self): ...
    def SetTraining(self, flag: bool): ...


@runtime_checkable
class Cacheable(Protocol):
    """A parametrized module whose computed weight can be held across several forward calls
    (nn/parametrize_generic.go:155)."""
    def Cached(self, *a, **kw): ...


# callback signatures (nn/hooks.go:43-54, nn/loss.go:457)
ForwardPreHook = Callable[[Module, torch.Tensor], Optional[torch.Tensor]]
ForwardHook = Callable[[Module, torch.Tensor, torch.Tensor], Optional[torch.Tensor]]
BackwardHook = Callable[[Module, torch.Tensor], Optional[torch.Tensor]]
DistanceFunc = Callable[[torch.Tensor, torch.Tensor], torch.Tensor]

__all__ = ["Param", "LSTMState", "Reduction", "ReduceMean", "ReduceSum", "ReduceNone", "Base", "Child",
           "Cacheable", "ForwardPreHook", "ForwardHook", "BackwardHook", "DistanceFunc"]

"""Magnitude / random pruning with a mask registry (nn/prune/prune.go:56-336).

The registry is keyed by tensor identity and holds a snapshot of the original values plus a
cumulative 0/1 mask.  Pruning zeroes the masked entries in place; call ``Reapply`` after every
optimizer step (this replaces PyTorch's forward pre-hook); ``Remove`` makes the pruning
permanent by dropping the entry.  ``k = round(amount * n)`` entries (or slices) are pruned;
ties are broken by position (stable sort).
"""
from __future__ import annotations

import threading
from typing import Dict, Sequence

import torch

_mu = threading.Lock()
_registry: Dict[int, dict] = {}


def _n_to_prune(amount: float, n: int) -> int:
    if not 0.0 <= amount <= 1.0:
        raise ValueError("prune: amount must be in [0, 1]")
    return min(max(int(round(amount * n)), 0), n)


@torch.no_grad()
def Prune(p: torch.Tensor, mask: torch.Tensor) -> None:
    mask = torch.as_tensor(mask, device=p.device).reshape(-1)
    if mask.numel() != p.numel():
        raise ValueError(f"prune: mask length {mask.numel()} does not match tensor numel {p.numel()}")
    with _mu:
        e = _registry.get(id(p))
        if e is None:
            e = {"tensor": p, "orig": p.detach().clone(), "mask": torch.ones(p.numel(), dtype=torch.bool, device=p.device)}
            _registry[id(p)] = e
        e["mask"] &= mask != 0
        p.data.reshape(-1)[~e["mask"]] = 0


@torch.no_grad()
def Reapply(*params: torch.Tensor) -> None:
    with _mu:
        for p in params:
            e = _registry.get(id(p))
            if e is not None:
                p.data.reshape(-1)[~e["mask"]] = 0


def Remove(p: torch.Tensor) -> None:
    with _mu:
        _registry.pop(id(p), None)


def IsPruned(p: torch.Tensor) -> bool:
    with _mu:
        return id(p) in _registry


def Mask(p: torch.Tensor):
    with _mu:
        e = _registry.get(id(p))
        return None if e is None else e["mask"].reshape(p.shape).to(p.dtype).clone()


def Orig(p: torch.Tensor):
    with _mu:
        e = _registry.get(id(p))
        return None if e is None else e["orig"].clone()


def Identity(p: torch.Tensor) -> None:
    Prune(p, torch.ones(p.numel()))


def CustomFromMask(p: torch.Tensor, mask) -> None:
    Prune(p, mask)


def RandomUnstructured(p: torch.Tensor, amount: float, seed: int = 0) -> None:
    n = p.numel()
    k = _n_to_prune(amount, n)
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(n, generator=g)
    mask = torch.ones(n)
    mask[perm[:k]] = 0
    Prune(p, mask)


def L1Unstructured(p: torch.Tensor, amount: float) -> None:
    n = p.numel()
    k = _n_to_prune(amount, n)
    order = torch.sort(p.detach().abs().reshape(-1).double().cpu(), stable=True).indices
    mask = torch.ones(n)
    mask[order[:k]] = 0
    Prune(p, mask)


def _structured_mask(p, dim, slices):
    mask = torch.ones_like(p, dtype=torch.float32)
    if len(slices):
        mask.index_fill_(dim, torch.as_tensor(slices, device=p.device, dtype=torch.long), 0.0)
    return mask.reshape(-1)


def LnStructured(p: torch.Tensor, amount: float, n: float, dim: int) -> None:
    dim = dim % p.dim()
    size = p.shape[dim]
    k = _n_to_prune(amount, size)
    flat = p.detach().double().movedim(dim, 0).reshape(size, -1).abs()
    norms = flat.max(1).values if n == float("inf") else flat.pow(n).sum(1).pow(1.0 / n)
    order = torch.sort(norms.cpu(), stable=True).indices
    Prune(p, _structured_mask(p, dim, order[:k].tolist()))


def RandomStructured(p: torch.Tensor, amount: float, dim: int, seed: int = 0) -> None:
    dim = dim % p.dim()
    size = p.shape[dim]
    k = _n_to_prune(amount, size)
    g = torch.Generator().manual_seed(seed)
    Prune(p, _structured_mask(p, dim, torch.randperm(size, generator=g)[:k].tolist()))


def GlobalUnstructured(params: Sequence[torch.Tensor], amount: float) -> None:
    total = sum(p.numel() for p in params)
    k = _n_to_prune(amount, total)
    allv = torch.cat([p.detach().abs().reshape(-1).double().cpu() for p in params])
    order = torch.sort(allv, stable=True).indices
    gmask = torch.ones(total)
    gmask[order[:k]] = 0
    off = 0
    for p in params:
        Prune(p, gmask[off:off + p.numel()])
        off += p.numel()

"""Embedding and EmbeddingBag (nn/embedding.go:45-429).  Weights ~ N(0, 1)."""
from __future__ import annotations

from typing import Optional

import torch

from ..ops.embedding import embedding as _embedding
from .module import Module


class Embedding(Module):
    def __init__(self, num_embeddings: int, embedding_dim: int, padding_idx: Optional[int] = None,
                 max_norm: Optional[float] = None, norm_type: float = 2.0, *, dtype=torch.float32,
                 device=None):
        super().__init__()
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.padding_idx, self.max_norm, self.norm_type = padding_idx, max_norm, norm_type
        w = torch.empty(num_embeddings, embedding_dim, dtype=torch.float32).normal_(0, 1)
        if padding_idx is not None:
            w[padding_idx].zero_()
        self.weight = torch.nn.Parameter(w.to(dtype=dtype, device=device))

    def forward(self, idx):
        if self.max_norm is not None:
            with torch.no_grad():
                rows = torch.unique(idx.reshape(-1).long())
                w = self.weight.data[rows]
                w = w if w.dtype == torch.float64 else w.float()
                n = w.norm(self.norm_type, dim=1, keepdim=True)
                scale = torch.where(n > self.max_norm, self.max_norm / (n + 1e-7), torch.ones_like(n))
                self.weight.data[rows] = (w * scale).to(self.weight.dtype)
        return _embedding(self.weight, idx, self.padding_idx)


class EmbeddingBag(Module):
    """Bags of embeddings reduced by sum / mean / max.  ``forward(idx, offsets)`` takes a
    flat index vector and bag start offsets (``offsets[0] == 0``, non-decreasing);
    ``Forward2D`` takes (bags, bag_len).  Empty or all-padding bags give a zero row."""

    def __init__(self, num_embeddings: int, embedding_dim: int, mode: str = "mean",
                 padding_idx: Optional[int] = None, max_norm: Optional[float] = None, norm_type: float = 2.0, *,
                 dtype=torch.float32, device=None):
        super().__init__()
        if mode not in ("sum", "mean", "max"):
            raise ValueError("nn.EmbeddingBag: mode must be sum, mean or max")
        self.mode, self.padding_idx = mode, padding_idx
        self.max_norm, self.norm_type = max_norm, norm_type
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        w = torch.empty(num_embeddings, embedding_dim, dtype=torch.float32).normal_(0, 1)
        if padding_idx is not None:
            w[padding_idx].zero_()
        self.weight = torch.nn.Parameter(w.to(dtype=dtype, device=device))

    def _renorm(self, idx):
        """Rows that are looked up and whose norm exceeds ``max_norm`` are rescaled in place, as
        in ``Embedding`` (nn/embedding.go:90-106)."""
        if self.max_norm is None:
            return
        with torch.no_grad():
            rows = torch.unique(idx.reshape(-1).long())
            w = self.weight.data[rows]
            w = w if w.dtype == torch.float64 else w.float()
            n = w.norm(self.norm_type, dim=1, keepdim=True)
            scale = torch.where(n > self.max_norm, self.max_norm / (n + 1e-7), torch.ones_like(n))
            self.weight.data[rows] = (w * scale).to(self.weight.dtype)

    def forward(self, idx, offsets=None):
        self._renorm(idx)
        if offsets is None:
            return self.Forward2D(idx)
        idx = idx.reshape(-1).long()
        offsets = offsets.reshape(-1).long()
        if offsets.numel() == 0 or int(offsets[0]) != 0 or bool((offsets[1:] < offsets[:-1]).any()):
            raise ValueError("nn.EmbeddingBag: offsets must start at 0 and be non-decreasing")
        n = idx.numel()
        nb = offsets.numel()
        bag_of = torch.bucketize(torch.arange(n, device=idx.device), offsets, right=True) - 1
        rows = _embedding(self.weight, idx, self.padding_idx)
        keep = torch.ones(n, dtype=rows.dtype, device=rows.device)
        if self.padding_idx is not None:
            keep = (idx != self.padding_idx).to(rows.dtype)
        if self.mode == "max":
            out = []
            ends = torch.cat([offsets[1:], offsets.new_tensor([n])])
            for b in range(nb):
                sel = rows[int(offsets[b]):int(ends[b])]
                k = keep[int(offsets[b]):int(ends[b])].bool()
                sel = sel[k]
                out.append(sel.max(0).values if sel.shape[0] else rows.new_zeros(self.embedding_dim))
            return torch.stack(out)
        # sum / mean as one product with a constant bag matrix, like the reference
        bagm = torch.zeros(nb, n, dtype=rows.dtype, device=rows.device)
        bagm[bag_of, torch.arange(n, device=idx.device)] = keep
        out = bagm @ rows
        if self.mode == "mean":
            cnt = bagm.sum(1, keepdim=True).clamp_min(1)
            out = out / cnt
        return out

    def Forward2D(self, idx2d):
        B, L = idx2d.shape
        offsets = torch.arange(0, B * L, L, device=idx2d.device)
        return self.forward(idx2d.reshape(-1), offsets)

"""Embedding lookup (row gather) with a deterministic scatter-add backward.

Reference: Embedding = IndexSelect with scatter-add backward
(tensor/ops_index.go:7-113, nn/embedding.go:108-126); ``padding_idx`` rows
receive no gradient.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import lib as _l


def _native(w):
    return w.is_cuda and w.dtype in (torch.bfloat16, torch.float16, torch.float32, torch.float64)


def gather_rows(weight: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    V, D = weight.shape
    flat = idx.reshape(-1).to(torch.int64).contiguous()
    out = torch.empty((flat.numel(), D), dtype=weight.dtype, device=weight.device)
    wc = weight.contiguous()
    _l.call("gb_gather_rows", _l.I(_l.dtype_code(weight.dtype)), _l.ptr(wc), _l.ptr(flat), _l.ptr(out),
            _l.L(flat.numel()), _l.I(D), _l.L(V), _l.stream_ptr())
    return out.reshape(*idx.shape, D)


def embedding_backward(dy: torch.Tensor, idx: torch.Tensor, V: int, padding_idx: Optional[int] = None,
                       out: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
    D = dy.shape[-1]
    flat = idx.reshape(-1).to(torch.int64).contiguous()
    dyc = dy.reshape(-1, D).contiguous()
    n = flat.numel()
    if out is None:
        out = torch.empty((V, D), dtype=dy.dtype, device=dy.device)
        accumulate = False
    ints = _l.lib().gb_embedding_bwd_scratch_ints
    ints.restype = _l.L
    scratch = torch.empty(int(ints(_l.L(n), _l.L(V))), dtype=torch.int32, device=dy.device)
    _l.call("gb_embedding_bwd", _l.I(_l.dtype_code(dy.dtype)), _l.I(_l.dtype_code(out.dtype)), _l.ptr(dyc),
            _l.ptr(flat), _l.ptr(out), _l.L(n), _l.I(D), _l.L(V),
            _l.L(padding_idx if padding_idx is not None else -1), _l.I(int(accumulate)), _l.ptr(scratch),
            _l.stream_ptr())
    return out


class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, weight, idx, padding_idx):
        ctx.save_for_backward(idx)
        ctx.V, ctx.padding_idx = weight.shape[0], padding_idx
        ctx.param = weight
        return gather_rows(weight, idx)

    @staticmethod
    def backward(ctx, dy):
        (idx,) = ctx.saved_tensors
        sink = getattr(ctx.param, "_gb_sink", None)
        if sink is not None:
            # written straight into the data-parallel bucket (overwrite on first use)
            buf, fresh = sink.target(ctx.param)
            embedding_backward(dy, idx, ctx.V, ctx.padding_idx, out=buf.view(ctx.param.shape),
                               accumulate=not fresh)
            sink.ready(ctx.param)
            return None, None, None
        return embedding_backward(dy, idx, ctx.V, ctx.padding_idx), None, None


def embedding(weight: torch.Tensor, idx: torch.Tensor, padding_idx: Optional[int] = None) -> torch.Tensor:
    if _native(weight):
        return _Embedding.apply(weight, idx, padding_idx)
    if weight.is_cuda:
        raise TypeError(f"embedding: no CUDA kernel for dtype {weight.dtype}")
    return torch.nn.functional.embedding(idx.long(), weight, padding_idx=padding_idx)

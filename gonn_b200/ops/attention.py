"""Fused attention: ``softmax(scale * Q K^T [+ causal mask]) V`` without the S x S matrix.

On CUDA with bf16/fp16 inputs and head_dim 64 or 128 this runs the tcgen05
flash-attention kernels (csrc/flash_attn.cu), forward and backward.  Otherwise
(CPU, fp32/fp64, other head sizes) the same math is evaluated with tensor ops,
using the reference's conventions: scale 1/sqrt(D) and an additive causal mask
of -1e30 (nn/attention.go:124-147, 185-196).

Tensors use the ``(B, S, H, D)`` layout ("bshd"); any strides with a contiguous
last dimension are accepted, so the q/k/v slices of a fused QKV projection can be
passed without copies.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import lib as _l


def attention_ref(q, k, v, causal: bool = False, scale: Optional[float] = None):
    """Oracle: materialised scores, additive -1e30 mask, softmax over keys. bshd layout."""
    B, Sq, H, D = q.shape
    Sk = k.shape[1]
    scale = (1.0 / math.sqrt(D)) if scale is None else scale
    ct = torch.float64 if q.dtype == torch.float64 else torch.float32
    qf, kf, vf = (t.to(ct).permute(0, 2, 1, 3) for t in (q, k, v))
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        mask = torch.triu(torch.ones(Sq, Sk, dtype=torch.bool, device=q.device), diagonal=1)
        s = s + mask.to(ct) * (-1e30)
    p = torch.softmax(s, dim=-1)
    o = torch.matmul(p, vf)
    return o.permute(0, 2, 1, 3).to(q.dtype)


def _strides3(t):
    return [t.stride(0), t.stride(1), t.stride(2)]


def _kernel_ok(q, k, v) -> bool:
    if not q.is_cuda or q.dtype not in (torch.bfloat16, torch.float16):
        return False
    if k.dtype != q.dtype or v.dtype != q.dtype:
        return False
    D = q.shape[-1]
    return D in (64, 128)


def _tma_ready(t):
    """TMA needs unit inner stride, 16-byte aligned base and strides."""
    if t.stride(-1) != 1 or t.data_ptr() % 16 or any(s % 8 for s in t.stride()[:-1]):
        return t.contiguous()
    return t


def flash_fwd(q, k, v, causal: bool, scale: float):
    """Returns (out, lse); out is contiguous (B,Sq,H,D), lse is (B,H,Sq) fp32."""
    q, k, v = _tma_ready(q), _tma_ready(k), _tma_ready(v)
    B, Sq, H, D = q.shape
    Sk = k.shape[1]
    out = torch.empty((B, Sq, H, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, H, Sq), dtype=torch.float32, device=q.device)
    I, L = _l.I, _l.L
    _l.call("gb_flash_fwd", I(_l.dtype_code(q.dtype)), _l.ptr(q), _l.ptr(k), _l.ptr(v), _l.ptr(out),
            _l.ptr(lse), I(B), I(H), I(Sq), I(Sk), I(D),
            *[L(s) for s in _strides3(q) + _strides3(k) + _strides3(v) + _strides3(out)],
            _l.F(scale), I(int(causal)), _l.stream_ptr())
    return out, lse


def flash_bwd(q, k, v, out, dout, lse, causal: bool, scale: float):
    q, k, v, dout = _tma_ready(q), _tma_ready(k), _tma_ready(v), _tma_ready(dout)
    B, Sq, H, D = q.shape
    Sk = k.shape[1]
    delta = torch.empty((B, H, Sq), dtype=torch.float32, device=q.device)
    I, L = _l.I, _l.L
    _l.call("gb_flash_delta", I(_l.dtype_code(q.dtype)), _l.ptr(out), _l.ptr(dout), _l.ptr(delta),
            I(B), I(H), I(Sq), I(D), *[L(s) for s in _strides3(out) + _strides3(dout)],
            _l.stream_ptr())
    # one allocation so that dq / dk / dv can be handed on as a fused (.., 3, H, D) gradient
    if Sq == Sk:
        dqkv = torch.empty((B, Sq, 3, H, D), dtype=q.dtype, device=q.device)
        dq, dk, dv = dqkv[:, :, 0], dqkv[:, :, 1], dqkv[:, :, 2]
    else:
        dqkv = None
        dq = torch.empty((B, Sq, H, D), dtype=q.dtype, device=q.device)
        dk = torch.empty((B, Sk, H, D), dtype=q.dtype, device=q.device)
        dv = torch.empty((B, Sk, H, D), dtype=q.dtype, device=q.device)
    strides = []
    for t in (q, k, v, dout, dq, dk, dv):
        strides += _strides3(t)
    arr = (_l.L * 21)(*strides)
    _l.call("gb_flash_bwd", I(_l.dtype_code(q.dtype)), _l.ptr(q), _l.ptr(k), _l.ptr(v), _l.ptr(dout),
            _l.ptr(lse), _l.ptr(delta), _l.ptr(dq), _l.ptr(dk), _l.ptr(dv), I(B), I(H), I(Sq),
            I(Sk), I(D), arr, _l.F(scale), I(int(causal)), _l.stream_ptr())
    return dq, dk, dv, dqkv


class _FlashAttn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale):
        out, lse = flash_fwd(q, k, v, causal, scale)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.causal, ctx.scale = causal, scale
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv, _ = flash_bwd(q, k, v, out, dout, lse, ctx.causal, ctx.scale)
        return dq, dk, dv, None, None


def flash_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = False,
                    scale: Optional[float] = None) -> torch.Tensor:
    """Attention over ``(B, S, H, D)`` tensors; differentiable."""
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("flash_attention: expected (B, S, H, D) tensors")
    D = q.shape[-1]
    scale = (1.0 / math.sqrt(D)) if scale is None else float(scale)
    if _kernel_ok(q, k, v) and not (causal and q.shape[1] != k.shape[1]):
        return _FlashAttn.apply(q, k, v, bool(causal), scale)
    return attention_ref(q, k, v, causal, scale)

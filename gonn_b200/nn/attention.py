"""MultiHeadAttention (nn/attention.go:13-341).

Children ``qproj`` / ``kproj`` / ``vproj`` / ``outproj`` are Linear layers with
bias; ``kdim`` / ``vdim`` set distinct key / value input sizes.  The core is
``softmax(Q K^T / sqrt(D) + mask) V`` with an additive -1e30 mask.

Self-attention on CUDA in bf16/fp16 takes the fused path: the three projections
run as one GEMM (their parameters are allocated back to back for that purpose)
followed by the flash-attention kernel; no (B, H, Tq, Tk) tensor exists.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..ops.attention import flash_attention, general_attention, general_ok, self_attention_qkv
from ..ops.softmax import softmax as _softmax
from .init import fan_in_uniform_
from .linear import Linear
from ..options import accepting_options as _accepting_options
from .module import Module


class MultiHeadAttention(Module):
    def __init__(self, embed_dim: int, num_heads: int, kdim: Optional[int] = None,
                 vdim: Optional[int] = None, *, dtype=torch.float32, device=None):
        super().__init__()
        if embed_dim % num_heads != 0:
            raise ValueError("MultiHeadAttention: embed_dim must be divisible by num_heads")
        kdim = embed_dim if kdim is None else kdim
        vdim = embed_dim if vdim is None else vdim
        if kdim < 1 or vdim < 1:
            raise ValueError("MultiHeadAttention: kdim and vdim must be >= 1")
        self.embed_dim, self.num_heads, self.head_dim = embed_dim, num_heads, embed_dim // num_heads
        self.kdim, self.vdim = kdim, vdim
        self.qproj = Linear(embed_dim, embed_dim, True, dtype=dtype, device=device)
        self.kproj = Linear(kdim, embed_dim, True, dtype=dtype, device=device)
        self.vproj = Linear(vdim, embed_dim, True, dtype=dtype, device=device)
        self.outproj = Linear(embed_dim, embed_dim, True, dtype=dtype, device=device)
        if kdim == embed_dim and vdim == embed_dim:
            self._pack_qkv()

    def _pack_qkv(self):
        """Re-homes the q/k/v parameters in one allocation each (weights, biases) so that
        the fused projection can address them as a single (3E, E) matrix."""
        E = self.embed_dim
        projs = (self.qproj, self.kproj, self.vproj)
        w = torch.cat([p.weight.data for p in projs], 0)
        b = torch.cat([p.bias.data for p in projs], 0)
        for i, p in enumerate(projs):
            p.weight.data = w[i * E:(i + 1) * E]
            p.bias.data = b[i * E:(i + 1) * E]

    def fuse_groups(self):
        """Parameter groups that must stay adjacent in memory when a wrapper re-homes
        parameters into flat buffers (keeps the one-GEMM QKV projection available)."""
        if self.kdim != self.embed_dim or self.vdim != self.embed_dim:
            return []
        return [[self.qproj.weight, self.kproj.weight, self.vproj.weight],
                [self.qproj.bias, self.kproj.bias, self.vproj.bias]]

    def _apply(self, fn, *a, **kw):
        # .to() / .cuda() / .bfloat16() re-allocate parameters one by one: pack again
        r = super()._apply(fn, *a, **kw)
        if self.kdim == self.embed_dim and self.vdim == self.embed_dim:
            self._pack_qkv()
        return r

    # -- forward variants -----------------------------------------------------------------
    def forward(self, q, k=None, v=None, causal: bool = False, residual=None, out_bias_grad: bool = True):
        """(B, Tq, E), (B, Tk, kdim), (B, Tk, vdim) -> (B, Tq, E).  ``residual`` is added in the
        output projection's epilogue; ``out_bias_grad=False`` leaves the gradient of the output
        projection's bias to the caller (``LayerNorm.fork`` produces it)."""
        k = q if k is None else k
        v = q if v is None else v
        self._check(q, k, v)
        if q is k and k is v:
            core = self_attention_qkv(q, self.qproj.weight, self.kproj.weight, self.vproj.weight,
                                      self.qproj.bias, self.kproj.bias, self.vproj.bias,
                                      self.num_heads, causal)
            if core is not None:
                return self.outproj(core, residual=residual, bias_grad=out_bias_grad)
        B, Tq, _ = q.shape
        Tk = k.shape[1]
        H, D = self.num_heads, self.head_dim
        Q = self.qproj(q).reshape(B, Tq, H, D)
        K = self.kproj(k).reshape(B, Tk, H, D)
        V = self.vproj(v).reshape(B, Tk, H, D)
        out = flash_attention(Q, K, V, causal=causal)
        return self.outproj(out.reshape(B, Tq, H * D), residual=residual, bias_grad=out_bias_grad)

    def ForwardFused(self, q, k=None, v=None, causal: bool = False):
        """Inference entry point of the reference (no tape): same math under no_grad."""
        with torch.no_grad():
            return self.forward(q, k, v, causal)

    @_accepting_options
    def ForwardMasked(self, q, k=None, v=None, causal: bool = False, attn_mask=None,
                      key_padding_mask=None, attn_dropout: float = 0.0):
        """General masks: ``attn_mask`` (Tq, Tk) additive float or bool (True = masked),
        ``key_padding_mask`` (B, Tk) bool (True = padded), dropout on the attention weights in
        training mode.  CUDA tensors run the fused general kernels (no score matrix); CPU
        tensors evaluate the same formula with tensor ops."""
        k = q if k is None else k
        v = q if v is None else v
        self._check(q, k, v)
        B, Tq, _ = q.shape
        Tk = k.shape[1]
        H, D = self.num_heads, self.head_dim
        if q.is_cuda:
            Q4 = self.qproj(q).reshape(B, Tq, H, D)
            K4 = self.kproj(k).reshape(B, Tk, H, D)
            V4 = self.vproj(v).reshape(B, Tk, H, D)
            if general_ok(Q4, K4, V4):
                pd = float(attn_dropout) if self.training else 0.0
                o = general_attention(Q4, K4, V4, causal, None, attn_mask, key_padding_mask, pd)
                return self.outproj(o.reshape(B, Tq, H * D))
        Q = self.qproj(q).reshape(B, Tq, H, D).permute(0, 2, 1, 3)
        K = self.kproj(k).reshape(B, Tk, H, D).permute(0, 2, 1, 3)
        V = self.vproj(v).reshape(B, Tk, H, D).permute(0, 2, 1, 3)
        ct = torch.float64 if q.dtype == torch.float64 else torch.float32     # 16-bit inputs widen to fp32
        s = torch.matmul(Q.to(ct), K.to(ct).transpose(-1, -2)) / math.sqrt(D)
        neg = -1e30
        if causal:
            s = s + torch.triu(torch.ones(Tq, Tk, device=s.device), 1)[None, None] * neg
        if attn_mask is not None:
            m = attn_mask.to(s.device)
            s = s + (m.to(ct) * neg if m.dtype == torch.bool else m.to(ct))[None, None]
        if key_padding_mask is not None:
            s = s + key_padding_mask.to(s.device).to(ct)[:, None, None, :] * neg
        p = _softmax(s, -1)
        if attn_dropout > 0 and self.training:
            p = torch.nn.functional.dropout(p, attn_dropout)
        o = torch.matmul(p, V.to(ct)).to(q.dtype).permute(0, 2, 1, 3).reshape(B, Tq, H * D)
        return self.outproj(o)

    def _check(self, q, k, v):
        if q.shape[-1] != self.embed_dim or k.shape[-1] != self.kdim or v.shape[-1] != self.vdim:
            raise ValueError("MultiHeadAttention: q/k/v feature sizes do not match embed_dim/kdim/vdim")
        if k.shape[1] != v.shape[1]:
            raise ValueError("MultiHeadAttention: k and v must have the same length")

"""Language models composed from the nn layers.

``TransformerLM``: token + position embeddings, N pre-LayerNorm encoder layers
with causal self-attention and a GELU feed-forward, final LayerNorm, untied
vocabulary projection.  ``GPT``: decoder-only blocks with RMSNorm, causal
attention and a GELU feed-forward.  Parameter names follow the reference's
naming contract for the layers they reuse (``layers.N.attn.qproj.weight``, ...).
"""
from __future__ import annotations

import torch

from ..nn.activation import GELU
from ..nn.attention import MultiHeadAttention
from ..nn.embedding import Embedding
from ..nn.linear import Linear
from ..nn.module import Module, ModuleList
from ..nn.norm import LayerNorm, RMSNorm
from ..nn.transformer import TransformerEncoderLayer
from ..ops.elementwise import binary as _binary
from ..ops.linear import feed_forward as _feed_forward
from ..ops.softmax import cross_entropy


class TransformerLM(Module):
    def __init__(self, vocab: int = 32000, d_model: int = 768, n_layers: int = 12, n_heads: int = 12,
                 d_ff: int = 3072, max_seq: int = 1024, *, dtype=torch.float32, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.vocab, self.d_model, self.max_seq = vocab, d_model, max_seq
        self.tok = Embedding(vocab, d_model, **kw)
        self.pos = Embedding(max_seq, d_model, **kw)
        self.layers = ModuleList([
            TransformerEncoderLayer(d_model, n_heads, d_ff, pre_norm=True, activation=GELU(), causal=True, **kw)
            for _ in range(n_layers)])
        self.norm = LayerNorm(d_model, **kw)
        self.head = Linear(d_model, vocab, bias=False, **kw)
        with torch.no_grad():
            self.tok.weight.mul_(0.02)
            self.pos.weight.mul_(0.02)

    def forward(self, ids):
        B, S = ids.shape
        pos = torch.arange(S, device=ids.device)
        x = _binary("add", self.tok(ids), self.pos(pos)[None])
        for l in self.layers:
            x = l(x)
        return self.head(self.norm(x))

    def loss(self, ids, targets):
        """Mean next-token cross-entropy; the logits' gradient overwrites the logits."""
        logits = self.forward(ids)
        return cross_entropy(logits.reshape(-1, self.vocab), targets.reshape(-1), inplace_backward=True,
                             consume_logits=True)


class GPTBlock(Module):
    def __init__(self, d_model: int, n_heads: int, d_ff: int, *, dtype=torch.float32, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.norm1 = RMSNorm(d_model, **kw)
        self.attn = MultiHeadAttention(d_model, n_heads, **kw)
        self.norm2 = RMSNorm(d_model, **kw)
        self.ff1 = Linear(d_model, d_ff, True, **kw)
        self.ff2 = Linear(d_ff, d_model, True, **kw)

    def forward(self, x):
        f1 = self.norm1.fork(x, self.attn.outproj.bias) if torch.is_grad_enabled() else None
        if f1 is not None:
            x = self.attn(f1[0], f1[0], f1[0], True, residual=f1[1], out_bias_grad=False)
        else:
            n = self.norm1(x)
            x = self.attn(n, n, n, True, residual=x)
        f2 = self.norm2.fork(x, self.ff2.bias) if torch.is_grad_enabled() else None
        if f2 is not None:
            return _feed_forward(f2[0], self.ff1.weight, self.ff1.bias, self.ff2.weight, self.ff2.bias,
                                 "gelu", f2[1], False)
        return _feed_forward(self.norm2(x), self.ff1.weight, self.ff1.bias, self.ff2.weight, self.ff2.bias,
                             "gelu", x)


class GPT(Module):
    """Decoder-only LM: 24 x (2048, 16 heads, 8192) with vocab 50304 is the 1.3 B config."""

    def __init__(self, vocab: int = 50304, d_model: int = 2048, n_layers: int = 24, n_heads: int = 16,
                 d_ff: int = 8192, max_seq: int = 2048, *, dtype=torch.float32, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.vocab, self.d_model, self.max_seq = vocab, d_model, max_seq
        self.tok = Embedding(vocab, d_model, **kw)
        self.pos = Embedding(max_seq, d_model, **kw)
        self.layers = ModuleList([GPTBlock(d_model, n_heads, d_ff, **kw) for _ in range(n_layers)])
        self.norm = RMSNorm(d_model, **kw)
        self.head = Linear(d_model, vocab, bias=False, **kw)
        with torch.no_grad():
            self.tok.weight.mul_(0.02)
            self.pos.weight.mul_(0.02)

    def forward(self, ids):
        B, S = ids.shape
        pos = torch.arange(S, device=ids.device)
        x = _binary("add", self.tok(ids), self.pos(pos)[None])
        for l in self.layers:
            x = l(x)
        return self.head(self.norm(x))

    def loss(self, ids, targets):
        logits = self.forward(ids)
        return cross_entropy(logits.reshape(-1, self.vocab), targets.reshape(-1), inplace_backward=True,
                             consume_logits=True)

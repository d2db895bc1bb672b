"""Transformer layers (nn/transformer.go:12-269, nn/transformer_full.go:13-47).

Child names follow the reference: encoder layer ``attn, norm1, ff1, ff2, norm2,
act, drop1, drop2, dropff``; decoder layer ``selfattn, norm1, crossattn, norm2,
ff1, ff2, norm3, ...``; stacks ``layers.N``.  Post-norm by default, pre-norm with
``pre_norm=True``; feed-forward activation defaults to ReLU.  The reference's
encoder self-attention is never causal; ``causal=True`` is an extension used to
build causal language models from encoder layers.
"""
from __future__ import annotations

import torch

from .activation import Activation, ReLU
from .attention import MultiHeadAttention
from .dropout import Dropout
from .linear import Linear
from .module import Module, ModuleList
from .norm import LayerNorm

_FUSABLE = {"relu": "relu", "gelu": "gelu", "geluexact": "geluexact"}


class TransformerEncoderLayer(Module):
    def __init__(self, embed_dim: int, num_heads: int, dim_ff: int, pre_norm: bool = False,
                 dropout: float = 0.0, activation: Activation = None, causal: bool = False, *,
                 dtype=torch.float32, device=None):
        super().__init__()
        self.pre_norm, self.causal = pre_norm, causal
        kw = dict(dtype=dtype, device=device)
        self.attn = MultiHeadAttention(embed_dim, num_heads, **kw)
        self.norm1 = LayerNorm(embed_dim, **kw)
        self.ff1 = Linear(embed_dim, dim_ff, True, **kw)
        self.ff2 = Linear(dim_ff, embed_dim, True, **kw)
        self.norm2 = LayerNorm(embed_dim, **kw)
        self.act = activation if activation is not None else ReLU()
        self.drop1 = Dropout(dropout)
        self.drop2 = Dropout(dropout)
        self.dropff = Dropout(dropout)

    def _ff(self, x, residual=None, bias2_grad: bool = True):
        kind = getattr(self.act, "kind", None)
        plain = not (self.training and self.dropff.p > 0)
        if kind in _FUSABLE and plain and type(self.act) is Activation:
            # activation fused into the first GEMM's epilogue, residual into the second's,
            # the activation's derivative into the second layer's data-gradient GEMM
            from ..ops.linear import feed_forward
            return feed_forward(x, self.ff1.weight, self.ff1.bias, self.ff2.weight, self.ff2.bias,
                                _FUSABLE[kind], residual, bias2_grad)
        if residual is not None and not (self.training and self.dropff.p > 0):
            return self.ff2(self.act(self.ff1(x)), residual=residual, bias_grad=bias2_grad)
        y = self.ff2(self.dropff(self.act(self.ff1(x))))
        return y if residual is None else residual + y

    def forward(self, x):
        nodrop = not (self.training and self.drop1.p > 0)
        if self.pre_norm:
            if nodrop:
                # x + attn(norm1(x)), then x + ff(norm2(x)): each norm also hands its input on, so
                # that its backward kernel adds the bypassing gradient and reduces the bias
                # gradient of the layer that closes the block
                f1 = self.norm1.fork(x, self.attn.outproj.bias) if torch.is_grad_enabled() else None
                if f1 is not None:
                    n, xp = f1
                    x = self.attn(n, n, n, self.causal, residual=xp, out_bias_grad=False)
                else:
                    n = self.norm1(x)
                    x = self.attn(n, n, n, self.causal, residual=x)
                f2 = self.norm2.fork(x, self.ff2.bias) if torch.is_grad_enabled() else None
                if f2 is not None:
                    return self._ff(f2[0], residual=f2[1], bias2_grad=False)
                return self._ff(self.norm2(x), residual=x)
            n = self.norm1(x)
            x = x + self.drop1(self.attn(n, n, n, self.causal))
            return x + self.drop2(self._ff(self.norm2(x)))
        if nodrop:
            x = self.norm1(self.attn(x, x, x, self.causal, residual=x))
            return self.norm2(self._ff(x, residual=x))
        x = self.norm1(x + self.drop1(self.attn(x, x, x, self.causal)))
        return self.norm2(x + self.drop2(self._ff(x)))


class TransformerEncoder(Module):
    def __init__(self, num_layers: int, embed_dim: int, num_heads: int, dim_ff: int, **opts):
        super().__init__()
        self.layers = ModuleList([TransformerEncoderLayer(embed_dim, num_heads, dim_ff, **opts)
                                  for _ in range(num_layers)])

    def forward(self, x):
        for l in self.layers:
            x = l(x)
        return x


class TransformerDecoderLayer(Module):
    """Causal self-attention, cross-attention over ``memory``, feed-forward."""

    def __init__(self, embed_dim: int, num_heads: int, dim_ff: int, pre_norm: bool = False,
                 dropout: float = 0.0, activation: Activation = None, *, dtype=torch.float32, device=None):
        super().__init__()
        self.pre_norm = pre_norm
        kw = dict(dtype=dtype, device=device)
        self.selfattn = MultiHeadAttention(embed_dim, num_heads, **kw)
        self.norm1 = LayerNorm(embed_dim, **kw)
        self.crossattn = MultiHeadAttention(embed_dim, num_heads, **kw)
        self.norm2 = LayerNorm(embed_dim, **kw)
        self.ff1 = Linear(embed_dim, dim_ff, True, **kw)
        self.ff2 = Linear(dim_ff, embed_dim, True, **kw)
        self.norm3 = LayerNorm(embed_dim, **kw)
        self.act = activation if activation is not None else ReLU()
        self.drop1 = Dropout(dropout)
        self.drop2 = Dropout(dropout)
        self.drop3 = Dropout(dropout)
        self.dropff = Dropout(dropout)

    def _ff(self, x):
        return self.ff2(self.dropff(self.act(self.ff1(x))))

    def forward(self, tgt, memory):
        if self.pre_norm:
            n = self.norm1(tgt)
            x = tgt + self.drop1(self.selfattn(n, n, n, True))
            n = self.norm2(x)
            x = x + self.drop2(self.crossattn(n, memory, memory, False))
            return x + self.drop3(self._ff(self.norm3(x)))
        x = self.norm1(tgt + self.drop1(self.selfattn(tgt, tgt, tgt, True)))
        x = self.norm2(x + self.drop2(self.crossattn(x, memory, memory, False)))
        return self.norm3(x + self.drop3(self._ff(x)))

    def ForwardModule(self, x):
        """Single-input form: the layer attends to its own input as memory."""
        return self.forward(x, x)


class TransformerDecoder(Module):
    def __init__(self, num_layers: int, embed_dim: int, num_heads: int, dim_ff: int, **opts):
        super().__init__()
        self.layers = ModuleList([TransformerDecoderLayer(embed_dim, num_heads, dim_ff, **opts)
                                  for _ in range(num_layers)])

    def forward(self, tgt, memory):
        for l in self.layers:
            tgt = l(tgt, memory)
        return tgt


class Transformer(Module):
    """Encoder-decoder with final LayerNorms ``encnorm`` / ``decnorm``."""

    def __init__(self, embed_dim: int, num_heads: int, num_enc: int, num_dec: int, dim_ff: int, **opts):
        super().__init__()
        self.encoder = TransformerEncoder(num_enc, embed_dim, num_heads, dim_ff, **opts)
        self.decoder = TransformerDecoder(num_dec, embed_dim, num_heads, dim_ff, **opts)
        kw = {k: opts[k] for k in ("dtype", "device") if k in opts}
        self.encnorm = LayerNorm(embed_dim, **kw)
        self.decnorm = LayerNorm(embed_dim, **kw)

    def forward(self, src, tgt):
        mem = self.encnorm(self.encoder(src))
        return self.decnorm(self.decoder(tgt, mem))

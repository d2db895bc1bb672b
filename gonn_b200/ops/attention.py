"""Fused attention: ``softmax(scale * Q K^T [+ causal mask]) V`` without the S x S matrix.

On CUDA with bf16/fp16 inputs and a head size that is a multiple of 8 (at most 128)
this runs the tcgen05 flash-attention kernels (csrc/flash_attn.cu), forward and
backward.  Masks (additive or boolean, key padding), attention dropout, fp32 / fp64
tensors and other head sizes up to 128 run the general fused kernels
(csrc/attn_general.cu), which keep no score matrix either.  On CPU the same math is
evaluated with tensor ops, using the reference's conventions: scale 1/sqrt(D) and an
additive mask of -1e30 (nn/attention.go:124-147, 185-196, 199-341).

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


def masked_attention_ref(q, k, v, causal=False, scale=None, attn_mask=None, key_padding_mask=None,
                         keep=None, p_drop: float = 0.0):
    """Oracle of the general path.  ``attn_mask``: additive float (Tq, Tk); ``key_padding_mask``: bool
    (B, Tk), True = padded; ``keep``: bool (B, H, Tq, Tk) dropout keep-mask (with ``p_drop``)."""
    B, Sq, H, D = q.shape
    Sk = k.shape[1]
    scale = (1.0 / math.sqrt(D)) if scale is None else scale
    ct = torch.float64 if q.dtype == torch.float64 else torch.float32
    qf, kf, vf = (t.to(ct).permute(0, 2, 1, 3) for t in (q, k, v))
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        s = s + torch.triu(torch.ones(Sq, Sk, dtype=torch.bool, device=q.device), diagonal=1).to(ct) * (-1e30)
    if attn_mask is not None:
        s = s + attn_mask.to(ct)[None, None]
    if key_padding_mask is not None:
        s = s + key_padding_mask.to(ct)[:, None, None, :] * (-1e30)
    p = torch.softmax(s, dim=-1)
    if keep is not None:
        p = p * keep.to(ct) / (1.0 - p_drop)
    return torch.matmul(p, vf).permute(0, 2, 1, 3).to(q.dtype)


def _general_call(mode, tensors, lse, delta, B, H, Tq, Tk, D, scale, causal, mask, kpm, p_drop, seed):
    import ctypes
    dt = None
    ptrs, strides = [], []
    for t in tensors:
        if t is None:
            ptrs.append(None)
            strides += [0, 0, 0]
        else:
            dt = t.dtype
            ptrs.append(t.data_ptr())
            strides += _strides3(t)
    parr = (ctypes.c_void_p * 8)(*ptrs)
    sarr = (_l.L * 24)(*strides)
    _l.call("gb_attn_general", _l.I(mode), _l.I(_l.dtype_code(dt)), parr, sarr, _l.ptr(lse), _l.ptr(delta), _l.I(B),
            _l.I(H), _l.I(Tq), _l.I(Tk), _l.I(D), _l.D(scale), _l.I(int(causal)), _l.ptr(mask), _l.ptr(kpm),
            _l.D(p_drop), _l.L(seed), _l.stream_ptr())


class _GeneralAttn(torch.autograd.Function):
    """The general fused kernels: forward, then dQ and dK/dV kernels that regenerate the dropout mask."""

    @staticmethod
    def forward(ctx, q, k, v, causal, scale, mask, kpm, p_drop, seed):
        q, k, v = (t if t.stride(-1) == 1 else t.contiguous() for t in (q, k, v))
        B, Tq, H, D = q.shape
        Tk = k.shape[1]
        out = torch.empty((B, Tq, H, D), dtype=q.dtype, device=q.device)
        st = torch.float64 if q.dtype == torch.float64 else torch.float32     # row statistics in the compute type
        lse = torch.empty((B, H, Tq), dtype=st, device=q.device)
        _general_call(0, [q, k, v, None, out, None, None, None], lse, None, B, H, Tq, Tk, D, scale, causal, mask, kpm,
                      p_drop, seed)
        ctx.save_for_backward(q, k, v, out, lse, mask, kpm)
        ctx.meta = (causal, scale, p_drop, seed)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse, mask, kpm = ctx.saved_tensors
        causal, scale, p_drop, seed = ctx.meta
        B, Tq, H, D = q.shape
        Tk = k.shape[1]
        dout = dout if dout.stride(-1) == 1 else dout.contiguous()
        delta = torch.empty((B, H, Tq), dtype=lse.dtype, device=q.device)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        ts = [q, k, v, dout, out, dq, dk, dv]
        common = (B, H, Tq, Tk, D, scale, causal, mask, kpm, p_drop, seed)
        _general_call(3, ts, lse, delta, *common)
        _general_call(1, ts, lse, delta, *common)
        _general_call(2, ts, lse, delta, *common)
        return dq, dk, dv, None, None, None, None, None, None


def general_fwd(q, k, v, causal: bool, scale: float):
    """(out, lse) from the general fused kernel; lse is (B, H, Tq) in the compute type."""
    q, k, v = (t if t.stride(-1) == 1 else t.contiguous() for t in (q, k, v))
    B, Tq, H, D = q.shape
    Tk = k.shape[1]
    out = torch.empty((B, Tq, H, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, H, Tq), dtype=torch.float64 if q.dtype == torch.float64 else torch.float32, device=q.device)
    _general_call(0, [q, k, v, None, out, None, None, None], lse, None, B, H, Tq, Tk, D, scale, causal, None, None, 0.0, 0)
    return out, lse


def general_bwd(q, k, v, out, dout, lse, causal: bool, scale: float):
    """(dq, dk, dv) from the general fused kernels, given the forward's output and lse."""
    q, k, v, out, dout = (t if t.stride(-1) == 1 else t.contiguous() for t in (q, k, v, out, dout))
    B, Tq, H, D = q.shape
    Tk = k.shape[1]
    st = torch.float64 if q.dtype == torch.float64 else torch.float32
    lse = lse.to(st).contiguous()
    delta = torch.empty((B, H, Tq), dtype=st, device=q.device)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    ts = [q, k, v, dout, out, dq, dk, dv]
    for mode in (3, 1, 2):
        _general_call(mode, ts, lse, delta, B, H, Tq, Tk, D, scale, causal, None, None, 0.0, 0)
    return dq, dk, dv


def general_attention(q, k, v, causal: bool = False, scale: Optional[float] = None, attn_mask=None,
                      key_padding_mask=None, dropout_p: float = 0.0, seed: Optional[int] = None):
    """Attention over ``(B, S, H, D)`` CUDA tensors with masks and dropout, fused (no score matrix).

    ``attn_mask``: (Tq, Tk) additive float, or bool with True = masked; ``key_padding_mask``: (B, Tk)
    bool, True = padded key; ``dropout_p``: probability of dropping an attention weight (the
    caller passes 0 in evaluation mode); ``seed`` fixes the dropout mask (drawn from torch's
    generator otherwise)."""
    B, Tq, H, D = q.shape
    Tk = k.shape[1]
    scale = (1.0 / math.sqrt(D)) if scale is None else float(scale)
    mask = None
    if attn_mask is not None:
        m = attn_mask.to(q.device)
        if tuple(m.shape) != (Tq, Tk):
            raise ValueError(f"attention: attn_mask must have shape ({Tq}, {Tk})")
        mask = (m.to(torch.float32) * -1e30 if m.dtype == torch.bool else m.to(torch.float32)).contiguous()
    kpm = None
    if key_padding_mask is not None:
        kp = key_padding_mask.to(q.device)
        if tuple(kp.shape) != (B, Tk):
            raise ValueError(f"attention: key_padding_mask must have shape ({B}, {Tk})")
        kpm = kp.to(torch.uint8).contiguous()
    if dropout_p > 0 and seed is None:
        seed = int(torch.randint(0, 2 ** 62, (1,)).item())
    return _GeneralAttn.apply(q, k, v, bool(causal), scale, mask, kpm, float(dropout_p), int(seed or 0))


def general_ok(q, k, v) -> bool:
    """True when the general fused kernels take these tensors (CUDA, one float dtype, head size <= 128)."""
    return (q.is_cuda and q.dtype in (torch.bfloat16, torch.float16, torch.float32, torch.float64)
            and k.dtype == q.dtype and v.dtype == q.dtype and q.shape[-1] <= 128)


def _kernel_ok(q, k, v) -> bool:
    if not q.is_cuda or q.dtype not in (torch.bfloat16, torch.float16):
        return False
    if k.dtype != q.dtype or v.dtype != q.dtype:
        return False
    D = q.shape[-1]
    return D % 8 == 0 and 8 <= D <= 128


def _tma_ready(t):
    """TMA needs unit inner stride, 16-byte aligned base and strides."""
    if t.stride(-1) != 1 or t.data_ptr() % 16 or any(s % 8 for s in t.stride()[:-1]):
        return t.contiguous()
    return t


def flash_fwd(q, k, v, causal: bool, scale: float, out=None):
    """Returns (out, lse); out is contiguous (B,Sq,H,D) unless a (B,Sq,H,D) view with unit inner
    stride and 16-byte aligned outer strides is passed in; lse is (B,H,Sq) fp32."""
    q, k, v = _tma_ready(q), _tma_ready(k), _tma_ready(v)
    B, Sq, H, D = q.shape
    Sk = k.shape[1]
    if out is None:
        out = torch.empty((B, Sq, H, D), dtype=q.dtype, device=q.device)
    elif (tuple(out.shape) != (B, Sq, H, D) or out.dtype != q.dtype or out.stride(-1) != 1
          or out.data_ptr() % 16 or any(s % 8 for s in out.stride()[:-1])):
        raise ValueError("flash_fwd: out must be a (B,Sq,H,D) view of the input dtype with unit inner "
                         "stride and outer strides that are multiples of 8 elements")
    lse = torch.empty((B, H, Sq), dtype=torch.float32, device=q.device)
    I, L = _l.I, _l.L
    _l.call("gb_flash_fwd", I(_l.dtype_code(q.dtype)), _l.ptr(q), _l.ptr(k), _l.ptr(v), _l.ptr(out),
            _l.ptr(lse), I(B), I(H), I(Sq), I(Sk), I(D),
            *[L(s) for s in _strides3(q) + _strides3(k) + _strides3(v) + _strides3(out)],
            _l.F(scale), I(int(causal)), _l.stream_ptr())
    return out, lse


# The backward keeps one workspace per device and stream for the spilled dS^T (see gb_flash_bwd_ws): with it the
# dK / dV kernel also writes dS and dQ is a single product read back from it, instead of a second pass
# that recomputes the scores.  Problems whose dS^T is larger than the limit take the two-pass path.
DS_SPILL_LIMIT_BYTES = 1 << 32          # the kernel's 32-bit offsets allow no more
_ds_ws = {}


def set_ds_spill_limit(nbytes: int) -> None:
    """Largest dS^T workspace the attention backward may use (0 turns the spill path off)."""
    global DS_SPILL_LIMIT_BYTES
    DS_SPILL_LIMIT_BYTES = min(int(nbytes), 1 << 32)
    _ds_ws.clear()


def _ds_workspace(device, need: int):
    if need <= 0 or need > DS_SPILL_LIMIT_BYTES:
        return None
    if torch.cuda.is_current_stream_capturing():
        # a captured graph keeps using the addresses it recorded: take the buffer from the graph's own
        # pool (which the graph keeps alive and reuses from layer to layer) instead of the cached one,
        # which a later, larger problem would replace
        return torch.empty(need, dtype=torch.uint8, device=device)
    key = (device, _l.current_stream_handle())     # one per stream: concurrent backward passes never share it
    ws = _ds_ws.get(key)
    if ws is None or ws.numel() < need:
        ws = _ds_ws[key] = torch.empty(need, dtype=torch.uint8, device=device)
    return ws


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
    need = (B * H * ((Sk + 127) // 128 * 128) * ((Sq + 127) // 128 * 128)) * 2
    ws = _ds_workspace(q.device, need)
    _l.call("gb_flash_bwd_ws", I(_l.dtype_code(q.dtype)), _l.ptr(q), _l.ptr(k), _l.ptr(v), _l.ptr(dout),
            _l.ptr(lse), _l.ptr(delta), _l.ptr(dq), _l.ptr(dk), _l.ptr(dv), I(B), I(H), I(Sq),
            I(Sk), I(D), arr, _l.F(scale), I(int(causal)), _l.ptr(ws), L(ws.numel() if ws is not None else 0),
            _l.stream_ptr())
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
    if general_ok(q, k, v):
        return general_attention(q, k, v, causal, scale)
    return attention_ref(q, k, v, causal, scale)


# ---------------------------------------------------------------------------
# Fused self-attention core: QKV projection (one GEMM) + flash attention.
# ---------------------------------------------------------------------------
def fused_view(parts):
    """If the tensors in ``parts`` lie back to back in one storage, returns one tensor that
    spans them (rows concatenated); otherwise None."""
    first = parts[0]
    if any(not p.is_contiguous() for p in parts):
        return None
    esz = first.element_size()
    ptr = first.data_ptr()
    for p in parts:
        if p.data_ptr() != ptr or p.dtype != first.dtype or p.shape[1:] != first.shape[1:]:
            return None
        ptr += p.numel() * esz
    rows = sum(p.shape[0] for p in parts)
    shape = (rows,) + tuple(first.shape[1:])
    strides = first.stride()
    try:
        return torch.as_strided(first, shape, strides)
    except RuntimeError:
        return None


def _emit_fused(params, grad_fn_into, grad_fn_new):
    """Writes one fused gradient for adjacent parameters, through sinks when present.

    ``grad_fn_into(out, beta)`` computes into a given buffer; ``grad_fn_new()`` returns
    a new tensor.  Returns the per-parameter gradients for autograd (None when sunk).
    """
    sinks = [getattr(p, "_gb_sink", None) for p in params]
    if all(s is not None for s in sinks):
        targets = [s.target(p) for s, p in zip(sinks, params)]
        bufs = [t[0].view(p.shape) for t, p in zip(targets, params)]
        fresh = [t[1] for t in targets]
        fused = fused_view(bufs) if len(set(fresh)) == 1 else None
        if fused is not None:
            grad_fn_into(fused, not fresh[0])
            for s, p in zip(sinks, params):
                s.ready(p)
            return [None] * len(params)
    g = grad_fn_new()
    outs, r0 = [], 0
    from .linear import emit_grad
    for p in params:
        outs.append(emit_grad(p, g[r0:r0 + p.shape[0]]))
        r0 += p.shape[0]
    return outs


class _SelfAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, wq, wk, wv, bq, bk, bv, wqkv, bqkv, H, causal, scale):
        from .gemm import gemm
        B, S, E = x.shape
        D = E // H
        x2 = x.reshape(B * S, E)
        qkv = gemm(x2, wqkv, trans_b=True, bias=bqkv)          # (B*S, 3E)
        qkv5 = qkv.view(B, S, 3, H, D)
        out, lse = flash_fwd(qkv5[:, :, 0], qkv5[:, :, 1], qkv5[:, :, 2], causal, scale)
        ctx.save_for_backward(x2, wqkv, qkv, out, lse)
        ctx.params = (wq, wk, wv, bq, bk, bv)
        ctx.meta = (B, S, E, H, D, causal, scale)
        return out.view(B, S, E)

    @staticmethod
    def backward(ctx, dout):
        from .gemm import gemm
        from .reduce import column_sum
        x2, wqkv, qkv, out, lse = ctx.saved_tensors
        wq, wk, wv, bq, bk, bv = ctx.params
        B, S, E, H, D, causal, scale = ctx.meta
        qkv5 = qkv.view(B, S, 3, H, D)
        dq, dk, dv, dqkv = flash_bwd(qkv5[:, :, 0], qkv5[:, :, 1], qkv5[:, :, 2], out,
                                     dout.reshape(B, S, H, D), lse, causal, scale)
        d2 = dqkv.view(B * S, 3 * E)
        dx = gemm(d2, wqkv).view(B, S, E) if ctx.needs_input_grad[0] else None
        gw = _emit_fused([wq, wk, wv],
                         lambda o, beta: gemm(d2, x2, trans_a=True, out=o, beta=beta),
                         lambda: gemm(d2, x2, trans_a=True))
        if bq is not None:
            gb = _emit_fused([bq, bk, bv],
                             lambda o, beta: column_sum(d2, out=o, accumulate=beta),
                             lambda: column_sum(d2))
        else:
            gb = [None, None, None]
        return (dx, gw[0], gw[1], gw[2], gb[0], gb[1], gb[2], None, None, None, None, None)


def self_attention_qkv(x, wq, wk, wv, bq, bk, bv, num_heads: int, causal: bool, scale=None):
    """``flash(x Wq^T + bq, x Wk^T + bk, x Wv^T + bv)`` for (B, S, E) input.

    Takes the one-GEMM path when the three weights (and biases) are adjacent in memory,
    bf16/fp16 on CUDA and head_dim is 64 or 128; returns None when that path does not
    apply so that the caller can fall back to separate projections.
    """
    E = x.shape[-1]
    D = E // num_heads
    if not (x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and D % 8 == 0 and 8 <= D <= 128 and x.dim() == 3):
        return None
    wqkv = fused_view([wq, wk, wv])
    if wqkv is None:
        return None
    bqkv = None
    if bq is not None:
        bqkv = fused_view([bq, bk, bv])
        if bqkv is None:
            return None
    scale = (1.0 / math.sqrt(D)) if scale is None else float(scale)
    return _SelfAttention.apply(x, wq, wk, wv, bq, bk, bv, wqkv.detach(), None if bqkv is None else bqkv.detach(),
                                num_heads, bool(causal), scale)

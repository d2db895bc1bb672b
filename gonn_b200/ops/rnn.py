"""Fused gate arithmetic of the LSTM / GRU cells (kernels in ``csrc/rnn.cu``).

``lstm_gates(gates, c) -> (h', c')`` with gate order i, f, g, o and
``gru_gates(xg, hg, h) -> h'`` with gates r, z, n (nn/rnn.go:159-286 of the reference).
CUDA tensors of fp32 / fp16 / bf16 run one kernel per direction; other tensors take the
torch expression with the same formulas (the oracle of the tests).
"""
from __future__ import annotations

import torch

from .. import lib as _l

_KERNEL_DTYPES = (torch.float32, torch.float16, torch.bfloat16)


def _on_kernels(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype in _KERNEL_DTYPES


def lstm_gates_ref(gates, c):
    H = c.shape[-1]
    i, f = torch.sigmoid(gates[:, :H]), torch.sigmoid(gates[:, H:2 * H])
    g, o = torch.tanh(gates[:, 2 * H:3 * H]), torch.sigmoid(gates[:, 3 * H:])
    c_new = f * c + i * g
    return o * torch.tanh(c_new), c_new


def gru_gates_ref(xg, hg, h):
    H = h.shape[-1]
    r = torch.sigmoid(xg[:, :H] + hg[:, :H])
    z = torch.sigmoid(xg[:, H:2 * H] + hg[:, H:2 * H])
    n = torch.tanh(xg[:, 2 * H:] + r * hg[:, 2 * H:])
    return (1 - z) * n + z * h


class _LSTMGates(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gates, c):
        B, H = c.shape
        gates, c = gates.contiguous(), c.contiguous()
        h_new, c_new = torch.empty_like(c), torch.empty_like(c)
        act = torch.empty_like(gates)
        _l.call("gb_lstm_gates_fwd", _l.I(_l.dtype_code(c.dtype)), _l.ptr(gates), _l.ptr(c), _l.ptr(h_new),
                _l.ptr(c_new), _l.ptr(act), _l.L(B), _l.I(H), _l.stream_ptr())
        ctx.save_for_backward(act, c, c_new)
        return h_new, c_new

    @staticmethod
    def backward(ctx, dh, dc):
        act, c, c_new = ctx.saved_tensors
        B, H = c.shape
        dh = dh.contiguous() if dh is not None else None
        dc = dc.contiguous() if dc is not None else None
        dgates, dc_prev = torch.empty_like(act), torch.empty_like(c)
        _l.call("gb_lstm_gates_bwd", _l.I(_l.dtype_code(c.dtype)), _l.ptr(act), _l.ptr(c), _l.ptr(c_new),
                _l.ptr(dh), _l.ptr(dc), _l.ptr(dgates), _l.ptr(dc_prev), _l.L(B), _l.I(H), _l.stream_ptr())
        return dgates, dc_prev


class _GRUGates(torch.autograd.Function):
    @staticmethod
    def forward(ctx, xg, hg, h):
        B, H = h.shape
        xg, hg, h = xg.contiguous(), hg.contiguous(), h.contiguous()
        h_new = torch.empty_like(h)
        act = torch.empty((B, 4 * H), dtype=h.dtype, device=h.device)
        _l.call("gb_gru_gates_fwd", _l.I(_l.dtype_code(h.dtype)), _l.ptr(xg), _l.ptr(hg), _l.ptr(h),
                _l.ptr(h_new), _l.ptr(act), _l.L(B), _l.I(H), _l.stream_ptr())
        ctx.save_for_backward(act, h)
        return h_new

    @staticmethod
    def backward(ctx, dh):
        act, h = ctx.saved_tensors
        B, H = h.shape
        dh = dh.contiguous()
        dxg = torch.empty((B, 3 * H), dtype=h.dtype, device=h.device)
        dhg = torch.empty_like(dxg)
        dh_prev = torch.empty_like(h)
        _l.call("gb_gru_gates_bwd", _l.I(_l.dtype_code(h.dtype)), _l.ptr(act), _l.ptr(h), _l.ptr(dh),
                _l.ptr(dxg), _l.ptr(dhg), _l.ptr(dh_prev), _l.L(B), _l.I(H), _l.stream_ptr())
        return dxg, dhg, dh_prev


def lstm_gates(gates: torch.Tensor, c: torch.Tensor):
    """(h', c') from the (B, 4H) gate pre-activations and the cell state."""
    if _on_kernels(c) and gates.dtype == c.dtype:
        return _LSTMGates.apply(gates, c)
    return lstm_gates_ref(gates, c)


def gru_gates(xg: torch.Tensor, hg: torch.Tensor, h: torch.Tensor):
    """h' from the (B, 3H) input / hidden pre-activations and the previous state."""
    if _on_kernels(h) and xg.dtype == h.dtype and hg.dtype == h.dtype:
        return _GRUGates.apply(xg, hg, h)
    return gru_gates_ref(xg, hg, h)

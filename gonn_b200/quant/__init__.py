"""int8 quantisation: per-tensor and per-channel PTQ, dynamic / static quantised Linear on the
tcgen05 int8 GEMM, fake quantisation and QAT (quant/quant.go, perchannel.go, linear.go, qat.go).

Conventions of the reference: ``round`` is half away from zero, int8 clamp [-128, 127], weights
are symmetric in [-127, 127] (zero point 0), activations are affine with the range nudged to
include 0; a quantised Linear computes
``y = sx * sw[o] * (acc - zx * rowsum[o]) + b[o]`` from an int8 x int8 -> int32 product.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from .. import lib as _l
from ..nn.linear import Linear
from ..nn.module import Module

QMin, QMax = -128, 127
DefaultAveragingConstant = 0.01


def _round_half_away(x: torch.Tensor) -> torch.Tensor:
    return torch.sign(x) * torch.floor(x.abs() + 0.5)


def quantize_value(v: torch.Tensor, scale, zero_point) -> torch.Tensor:
    return torch.clamp(_round_half_away(v / scale) + zero_point, QMin, QMax)


def affine_qparams(min_val: float, max_val: float):
    mn, mx = min(0.0, float(min_val)), max(0.0, float(max_val))
    scale = (mx - mn) / float(QMax - QMin)
    if scale == 0:
        return 1.0, 0
    r = mn / scale
    zp = QMin - int(torch.sign(torch.tensor(r)) * torch.floor(torch.tensor(abs(r)) + 0.5))
    return scale, min(max(zp, QMin), QMax)


def symmetric_qparams(t: torch.Tensor) -> float:
    m = float(t.detach().abs().max()) if t.numel() else 0.0
    return 1.0 if m == 0 else m / QMax


def symmetric_range_scale(mn: float, mx: float) -> float:
    m = max(abs(mn), abs(mx))
    return 1.0 if m == 0 else m / QMax


@dataclass
class QTensor:
    Data: torch.Tensor      # int8
    Scale: float
    ZeroPoint: int
    Shape: tuple

    def Numel(self) -> int:
        return self.Data.numel()


def Quantize(t: torch.Tensor, scale: Optional[float] = None, zero_point: Optional[int] = None) -> QTensor:
    """Affine per-tensor quantisation; q-parameters from the tensor's min / max when not given."""
    if scale is None:
        scale, zero_point = affine_qparams(float(t.min()), float(t.max())) if t.numel() else (1.0, 0)
    q = quantize_value(t.detach().double(), scale, zero_point or 0).to(torch.int8)
    return QTensor(q, float(scale), int(zero_point or 0), tuple(t.shape))


def Dequantize(q: QTensor, dtype=torch.float64) -> torch.Tensor:
    return ((q.Data.to(torch.float64) - q.ZeroPoint) * q.Scale).to(dtype).reshape(q.Shape)


@dataclass
class QTensorPerChannel:
    Data: torch.Tensor
    Scales: torch.Tensor
    Axis: int
    Shape: tuple

    def Numel(self) -> int:
        return self.Data.numel()

    @property
    def ZeroPoints(self):
        """Per-channel zero points: all zero, the scheme is symmetric (quant/perchannel.go:12-20)."""
        return [0] * self.Scales.numel()

    def Channels(self) -> int:
        """Number of quantisation channels: the size of ``Axis`` (quant/perchannel.go:28-29)."""
        return self.Scales.numel()


def QuantizePerChannel(t: torch.Tensor, axis: int = 0) -> QTensorPerChannel:
    """Symmetric per-channel quantisation along ``axis`` (zero point 0)."""
    axis = axis % t.dim()
    tt = t.detach().double().movedim(axis, 0)
    m = tt.reshape(tt.shape[0], -1).abs().max(1).values
    scales = torch.where(m == 0, torch.ones_like(m), m / QMax)
    shape = [-1] + [1] * (tt.dim() - 1)
    q = quantize_value(tt, scales.reshape(shape), 0).to(torch.int8).movedim(0, axis)
    return QTensorPerChannel(q.contiguous(), scales, axis, tuple(t.shape))


def DequantizePerChannel(q: QTensorPerChannel, dtype=torch.float64) -> torch.Tensor:
    shape = [1] * len(q.Shape)
    shape[q.Axis] = -1
    return (q.Data.to(torch.float64) * q.Scales.reshape(shape)).to(dtype)


class MinMaxObserver:
    def __init__(self):
        self.Min = self.Max = 0.0
        self.seen = False

    def Observe(self, t: torch.Tensor):
        if t.numel() == 0:
            return
        mn, mx = float(t.min()), float(t.max())
        if not self.seen:
            self.Min, self.Max, self.seen = mn, mx, True
        else:
            self.Min, self.Max = min(self.Min, mn), max(self.Max, mx)

    def Seen(self):
        return self.seen

    def ComputeQParams(self):
        return affine_qparams(self.Min, self.Max) if self.seen else (1.0, 0)


class MovingAverageMinMaxObserver(MinMaxObserver):
    def __init__(self, momentum: float = 0.0):
        super().__init__()
        self.Momentum = momentum

    def Observe(self, t: torch.Tensor):
        if t.numel() == 0:
            return
        mn, mx = float(t.min()), float(t.max())
        if not self.seen:
            self.Min, self.Max, self.seen = mn, mx, True
            return
        c = self.Momentum or DefaultAveragingConstant
        self.Min = (1 - c) * self.Min + c * mn
        self.Max = (1 - c) * self.Max + c * mx


# ---------------------------------------------------------------------------------------
# quantised Linear
# ---------------------------------------------------------------------------------------
class _QLinearCore:
    """int8 weight (out, in), per-row scales, per-row sums, float bias."""

    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor], per_channel: bool):
        out_f, in_f = weight.shape
        self.in_features, self.out_features, self.per_channel = in_f, out_f, per_channel
        w = weight.detach().double()
        if per_channel:
            qc = QuantizePerChannel(w, 0)
            self.WScales, self.WQ = qc.Scales.clone(), qc.Data
        else:
            s = symmetric_qparams(w)
            self.WScales = torch.full((out_f,), s, dtype=torch.float64)
            self.WQ = quantize_value(w, s, 0).to(torch.int8)
        self.WRowSum = self.WQ.to(torch.int32).sum(1).to(torch.int32)
        self.Bias = bias.detach().double().clone() if bias is not None else None
        self._dev = {}

    def _device_state(self, device):
        st = self._dev.get(str(device))
        if st is None:
            kp = (self.in_features + 15) // 16 * 16
            wq = torch.zeros((self.out_features, kp), dtype=torch.int8, device=device)
            wq[:, :self.in_features] = self.WQ.to(device)
            st = dict(wq=wq, kp=kp, sw=self.WScales.to(device=device, dtype=torch.float32).contiguous(),
                      rs=self.WRowSum.to(device).contiguous(),
                      b=self.Bias.to(device=device, dtype=torch.float32).contiguous() if self.Bias is not None else None)
            self._dev[str(device)] = st
        return st

    def forward_host(self, x: torch.Tensor, sx: float, zx: int) -> torch.Tensor:
        """Reference evaluation: integer accumulation, then the dequantising formula."""
        x2 = x.reshape(-1, self.in_features).double()
        xq = quantize_value(x2, sx, zx).to(torch.int64)
        acc = xq @ self.WQ.to(torch.int64).t().to(xq.device)
        y = sx * self.WScales.to(x.device)[None] * (acc - zx * self.WRowSum.to(torch.int64).to(x.device)[None]).double()
        if self.Bias is not None:
            y = y + self.Bias.to(x.device)[None]
        return y.to(x.dtype).reshape(*x.shape[:-1], self.out_features)

    def forward_device(self, x: torch.Tensor, qp4: torch.Tensor, zp: torch.Tensor) -> torch.Tensor:
        """tcgen05 int8 GEMM; ``qp4`` = {min, max, scale, zp} and ``zp`` (int32) live on the device."""
        st = self._device_state(x.device)
        x2 = x.reshape(-1, self.in_features).contiguous()
        M = x2.shape[0]
        xq = torch.zeros((M, st["kp"]), dtype=torch.int8, device=x.device) if st["kp"] != self.in_features \
            else torch.empty((M, st["kp"]), dtype=torch.int8, device=x.device)
        _l.call("gb_q_quantize", _l.I(_l.dtype_code(x.dtype)), _l.ptr(x2), _l.ptr(xq), _l.L(M), _l.L(self.in_features),
                _l.L(st["kp"]), _l.ptr(qp4[2:]), _l.ptr(zp), _l.I(0), _l.stream_ptr())
        out_dt = x.dtype if x.dtype in (torch.bfloat16, torch.float16) else torch.float32
        y = torch.empty((M, self.out_features), dtype=out_dt, device=x.device)
        _l.call("gb_gemm_i8", _l.ptr(xq), _l.ptr(st["wq"]), _l.ptr(y), _l.ptr(st["b"]), _l.I(M), _l.I(self.out_features),
                _l.I(st["kp"]), _l.L(st["kp"]), _l.L(st["kp"]), _l.L(self.out_features), _l.ptr(qp4[2:]), _l.ptr(zp),
                _l.ptr(st["sw"]), _l.I(1), _l.ptr(st["rs"]), _l.I(_l.dtype_code(out_dt)), _l.stream_ptr())
        return y.to(x.dtype).reshape(*x.shape[:-1], self.out_features)


def _observe_device(x: torch.Tensor, symmetric: bool = False):
    n = _l.lib().gb_q_scratch_floats()
    scratch = torch.empty(n, dtype=torch.float32, device=x.device)
    qp4 = torch.empty(4, dtype=torch.float32, device=x.device)
    zp = torch.empty(1, dtype=torch.int32, device=x.device)
    xc = x.contiguous()
    _l.call("gb_q_observe", _l.I(_l.dtype_code(x.dtype)), _l.ptr(xc), _l.L(xc.numel()), _l.I(int(symmetric)),
            _l.ptr(scratch), _l.ptr(qp4), _l.ptr(zp), _l.stream_ptr())
    return qp4, zp


def _native(x):
    return x.is_cuda and x.dtype in (torch.bfloat16, torch.float16, torch.float32)


class DynamicLinear(Module):
    """Weights quantised once; the input's q-parameters are computed per call from its min / max
    (on the device for CUDA inputs: no host synchronisation).  Inference only."""

    def __init__(self, linear: Linear, per_channel_weights: bool = False):
        super().__init__()
        self.core = _QLinearCore(linear.weight, linear.bias, per_channel_weights)

    @torch.no_grad()
    def forward(self, x):
        if _native(x):
            qp4, zp = _observe_device(x)
            return self.core.forward_device(x, qp4, zp)
        sx, zx = affine_qparams(float(x.min()), float(x.max()))
        return self.core.forward_host(x, sx, zx)


class StaticLinear(Module):
    """Input q-parameters fixed by calibration (``Calibrate`` feeds a MinMaxObserver)."""

    def __init__(self, linear: Linear, per_channel_weights: bool = False, in_scale: float = 1.0,
                 in_zero_point: int = 0):
        super().__init__()
        self.core = _QLinearCore(linear.weight, linear.bias, per_channel_weights)
        self.InScale, self.InZeroPoint = float(in_scale), int(in_zero_point)
        self.observer = MinMaxObserver()
        self._qp_dev = {}

    def Calibrate(self, x: torch.Tensor):
        self.observer.Observe(x)
        self.InScale, self.InZeroPoint = self.observer.ComputeQParams()
        self._qp_dev.clear()

    @torch.no_grad()
    def forward(self, x):
        if _native(x):
            k = str(x.device)
            if k not in self._qp_dev:
                self._qp_dev[k] = (torch.tensor([0, 0, self.InScale, self.InZeroPoint], dtype=torch.float32, device=x.device),
                                   torch.tensor([self.InZeroPoint], dtype=torch.int32, device=x.device))
            return self.core.forward_device(x, *self._qp_dev[k])
        return self.core.forward_host(x, self.InScale, self.InZeroPoint)


def WithPerChannelWeights():
    return {"per_channel_weights": True}


# ---------------------------------------------------------------------------------------
# QAT
# ---------------------------------------------------------------------------------------
class _FakeQuantFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale, zp):
        if _native(x):
            qp = torch.tensor([scale, zp], dtype=torch.float32, device=x.device)
            xc = x.contiguous()
            y = torch.empty_like(xc)
            _l.call("gb_fake_quant", _l.I(0), _l.I(_l.dtype_code(x.dtype)), _l.ptr(xc), None, _l.ptr(y), _l.L(xc.numel()),
                    _l.ptr(qp), _l.stream_ptr())
            ctx.save_for_backward(xc, qp)
            ctx.dev = True
            return y
        ctx.dev = False
        ctx.save_for_backward(x)
        ctx.rng = ((QMin - zp) * scale, (QMax - zp) * scale)
        return ((quantize_value(x.double(), scale, zp) - zp) * scale).to(x.dtype)

    @staticmethod
    def backward(ctx, g):
        if ctx.dev:
            xc, qp = ctx.saved_tensors
            gc = g.contiguous()
            dx = torch.empty_like(xc)
            _l.call("gb_fake_quant", _l.I(1), _l.I(_l.dtype_code(xc.dtype)), _l.ptr(xc), _l.ptr(gc), _l.ptr(dx),
                    _l.L(xc.numel()), _l.ptr(qp), _l.stream_ptr())
            return dx, None, None
        (x,) = ctx.saved_tensors
        lo, hi = ctx.rng
        return g * ((x >= lo) & (x <= hi)).to(g.dtype), None, None


class FakeQuant(Module):
    """Simulated int8 quantisation with a clamped straight-through gradient.  Training updates a
    moving-average min / max observer and the q-parameters; evaluation freezes them."""

    def __init__(self, symmetric: bool = False):
        super().__init__()
        self.Observer = MovingAverageMinMaxObserver()
        self.Symmetric = symmetric
        self.Scale, self.ZeroPoint = 1.0, 0

    def QParams(self):
        return self.Scale, self.ZeroPoint

    def _compute(self):
        if not self.Observer.Seen():
            return 1.0, 0
        if self.Symmetric:
            return symmetric_range_scale(self.Observer.Min, self.Observer.Max), 0
        return affine_qparams(self.Observer.Min, self.Observer.Max)

    def forward(self, x):
        if self.training:
            self.Observer.Observe(x.detach())
            self.Scale, self.ZeroPoint = self._compute()
        return _FakeQuantFn.apply(x, float(self.Scale), int(self.ZeroPoint))


class QATLinear(Module):
    """Linear with fake-quantised weight (symmetric) and input (affine); children ``linear``,
    ``weight_fq``, ``input_fq``.  ``Convert()`` produces the StaticLinear that evaluation of this
    module simulates."""

    def __init__(self, linear: Linear):
        super().__init__()
        self.linear = linear
        self.weight_fq = FakeQuant(symmetric=True)
        self.input_fq = FakeQuant(symmetric=False)

    # exported fields of the reference's struct (quant/qat.go:170-180)
    L = property(lambda self: self.linear)
    WeightFQ = property(lambda self: self.weight_fq)
    InputFQ = property(lambda self: self.input_fq)

    def forward(self, x):
        from ..ops.linear import linear as _linear
        return _linear(self.input_fq(x), self.weight_fq(self.linear.weight), self.linear.bias)

    def Convert(self) -> StaticLinear:
        ws, _ = self.weight_fq.QParams()
        out = StaticLinear(self.linear, False, *self.input_fq.QParams())
        # use exactly the weight scale QAT trained with
        w = self.linear.weight.detach().double()
        out.core.WScales = torch.full((self.linear.out_features,), float(ws), dtype=torch.float64)
        out.core.WQ = quantize_value(w, float(ws), 0).to(torch.int8)
        out.core.WRowSum = out.core.WQ.to(torch.int32).sum(1).to(torch.int32)
        out.core._dev.clear()
        return out


# ---------------------------------------------------------------------------------------
# constructor spellings of the reference (quant/linear.go:163-207, quant/qat.go:114-200)
# ---------------------------------------------------------------------------------------
LinearOption = dict        # what WithPerChannelWeights() returns: keyword arguments of the layers


def _merge(opts) -> dict:
    kw = {}
    for o in opts:
        kw.update(o)
    return kw


def NewDynamicLinearFrom(l: Linear, *opts: LinearOption) -> DynamicLinear:
    return DynamicLinear(l, **_merge(opts))


def NewStaticLinearFrom(l: Linear, obs: MinMaxObserver, *opts: LinearOption) -> StaticLinear:
    """Input q-parameters taken from a calibrated observer."""
    scale, zp = obs.ComputeQParams()
    return StaticLinear(l, in_scale=scale, in_zero_point=zp, **_merge(opts))


def NewFakeQuant(symmetric: bool) -> FakeQuant:
    return FakeQuant(symmetric)


def NewQATLinearFrom(l: Linear) -> QATLinear:
    return QATLinear(l)

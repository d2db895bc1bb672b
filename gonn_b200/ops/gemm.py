"""GEMM front end: ``C = epilogue(alpha * op(A) @ op(B))`` with trans flags.

Mirrors the reference's backend contract ``Gemm(a, b, batch, m, k, n, transA,
transB)`` (backend/backend.go:61-78): row-major operands, contiguous batches,
``op(A)`` is (m,k) and is stored (k,m) when ``trans_a``.  On CUDA, bf16/fp16
operands run on the tcgen05 kernel (csrc/gemm.cu); fp64 on the double-precision
tensor-core kernel and fp32 as three bf16 planes per operand on tcgen05
(csrc/gemm_exact.cu), with the register-tiled SIMT kernel for small or unaligned
problems; on CPU the same contract is evaluated with torch as the oracle path.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import lib as _l

ACT = {None: 0, "none": 0, "relu": 1, "gelu": 2, "gelu_tanh": 2, "geluexact": 3, "gelu_erf": 3}
AUX = {None: 0, "none": 0, "add": 1, "store_pre": 2, "mul_dgelu": 3, "mul_dgelu_tanh": 3,
       "mul_drelu": 4, "mul_dgeluexact": 5, "mul_dgelu_erf": 5}


def _act_ref(x, act):
    a = ACT[act]
    if a == 1:
        return torch.relu(x)
    if a == 2:
        return torch.nn.functional.gelu(x, approximate="tanh")
    if a == 3:
        return torch.nn.functional.gelu(x)
    return x


def _dact_ref(pre, mode):
    pre = pre.detach().clone().requires_grad_(True)
    with torch.enable_grad():
        if mode == 3:
            y = torch.nn.functional.gelu(pre, approximate="tanh")
        elif mode == 5:
            y = torch.nn.functional.gelu(pre)
        else:
            y = torch.relu(pre)
        (g,) = torch.autograd.grad(y.sum(), pre)
    return g


_WS_BYTES = 256 << 20
_ws_cache = {}
_x3_cache = {}
_FP32_MODE = "bf16x3"


def set_fp32_gemm_mode(mode: str) -> str:
    """``"bf16x3"`` (default): large fp32 products run on the tensor cores as three bf16 planes
    per operand (error at the rounding level of an fp32 product); ``"simt"``: always the
    register-tiled fp32 FMA kernel.  Returns the previous mode."""
    global _FP32_MODE
    if mode not in ("bf16x3", "simt"):
        raise ValueError("fp32 GEMM mode must be 'bf16x3' or 'simt'")
    old, _FP32_MODE = _FP32_MODE, mode
    return old


def _x3_workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    key = (device.index, _l.current_stream_handle())
    buf = _x3_cache.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _x3_cache[key] = buf
    return buf


def _workspace(device: torch.device) -> torch.Tensor:
    """fp32 scratch for split-K partial products, one per (device, stream) so that launches
    on different streams never share it."""
    key = (device.index, _l.current_stream_handle())
    buf = _ws_cache.get(key)
    if buf is None:
        buf = torch.empty(_WS_BYTES, dtype=torch.uint8, device=device)
        _ws_cache[key] = buf
    return buf


def _gemm_ref(a, b, trans_a, trans_b, bias, act, aux, aux_mode, out_dtype, beta, out, alpha):
    """Oracle path (CPU, or any dtype the kernels do not take): fp32/fp64 math in torch."""
    ct = torch.float64 if a.dtype == torch.float64 else torch.float32
    A = a.to(ct).transpose(-1, -2) if trans_a else a.to(ct)
    B = b.to(ct).transpose(-1, -2) if trans_b else b.to(ct)
    v = torch.matmul(A, B)
    if alpha != 1.0:
        v = v * alpha
    if bias is not None:
        v = v + bias.to(ct)
    m = AUX[aux_mode] if aux is not None else 0
    if m == 2:
        aux.copy_(v.to(aux.dtype))
    v = _act_ref(v, act)
    if m == 1:
        v = v + aux.to(ct)
    elif m in (3, 4, 5):
        v = v * _dact_ref(aux.to(ct), m)
    if out is not None:
        if beta:
            v = v + out.to(ct)
        out.copy_(v.to(out.dtype))
        return out
    return v.to(out_dtype)


def _pad_last(t: torch.Tensor, mult: int) -> torch.Tensor:
    n = t.shape[-1]
    r = (-n) % mult
    if r == 0 and t.stride(-1) == 1 and t.stride(-2) % mult == 0 and t.data_ptr() % 16 == 0:
        return t
    out = t.new_zeros(*t.shape[:-1], n + r)
    out[..., :n] = t
    return out[..., :n]


def _row_major_2d(t: torch.Tensor):
    """Returns (tensor, ld) with unit inner stride; copies only when needed."""
    if t.stride(-1) != 1 or (t.shape[-2] > 1 and t.stride(-2) < t.shape[-1]):
        t = t.contiguous()
    ld = t.stride(-2) if t.shape[-2] > 1 else max(t.shape[-1], t.stride(-2))
    return t, ld


def gemm(a: torch.Tensor, b: torch.Tensor, *, trans_a: bool = False, trans_b: bool = False,
         bias: Optional[torch.Tensor] = None, act: Optional[str] = None,
         aux: Optional[torch.Tensor] = None, aux_mode: Optional[str] = None,
         out_dtype: Optional[torch.dtype] = None, beta: bool = False,
         out: Optional[torch.Tensor] = None, alpha: float = 1.0,
         force_bn: int = 0) -> torch.Tensor:
    """2-D or batched (3-D, equal or broadcast batch) GEMM with a fused epilogue.

    ``bias`` has length N.  ``aux`` is an (M,N) tensor whose role is given by
    ``aux_mode``: ``"add"`` (residual), ``"store_pre"`` (receives the
    pre-activation), ``"mul_dgelu"`` / ``"mul_drelu"`` / ``"mul_dgeluexact"``
    (multiplies the result by the activation derivative at ``aux``).  ``beta``
    accumulates onto ``out``.
    """
    if a.dim() not in (2, 3) or b.dim() not in (2, 3):
        raise ValueError("gemm: operands must be 2-D or 3-D")
    batched = a.dim() == 3 or b.dim() == 3
    M, K = (a.shape[-1], a.shape[-2]) if trans_a else (a.shape[-2], a.shape[-1])
    Kb, N = (b.shape[-1], b.shape[-2]) if trans_b else (b.shape[-2], b.shape[-1])
    if K != Kb:
        raise ValueError(f"gemm: inner dimensions differ ({K} vs {Kb})")
    batch = 1
    if batched:
        ba = a.shape[0] if a.dim() == 3 else 1
        bb = b.shape[0] if b.dim() == 3 else 1
        if ba != bb and 1 not in (ba, bb):
            raise ValueError(f"gemm: batch sizes differ ({ba} vs {bb})")
        batch = max(ba, bb)
    if out_dtype is None:
        out_dtype = out.dtype if out is not None else a.dtype
    native16 = a.is_cuda and a.dtype in (torch.bfloat16, torch.float16) and b.dtype == a.dtype
    native_simt = a.is_cuda and a.dtype in (torch.float32, torch.float64) and b.dtype == a.dtype
    if not (native16 or native_simt):
        if a.is_cuda:
            raise TypeError(f"gemm: no CUDA kernel for dtypes {a.dtype} x {b.dtype}")
        return _gemm_ref(a, b, trans_a, trans_b, bias, act, aux, aux_mode, out_dtype, beta, out,
                         alpha)

    oshape = (batch, M, N) if batched else (M, N)
    if out is None:
        out = torch.empty(oshape, dtype=out_dtype, device=a.device)
        beta = False
    elif tuple(out.shape) != oshape or out.stride(-1) != 1:
        raise ValueError(f"gemm: out has shape {tuple(out.shape)}, expected {oshape}")

    if native_simt:
        if bias is not None or ACT[act] or (aux is not None and AUX[aux_mode]):
            # exact-precision path: epilogue evaluated with tensor ops
            tmp = gemm(a, b, trans_a=trans_a, trans_b=trans_b, alpha=alpha)
            return _epilogue_torch(tmp, bias, act, aux, aux_mode, beta, out)
        a2, lda = _row_major_2d(a)
        b2, ldb = _row_major_2d(b)
        sA = a2.stride(0) if a2.dim() == 3 and a2.shape[0] > 1 else 0
        sB = b2.stride(0) if b2.dim() == 3 and b2.shape[0] > 1 else 0
        sC = out.stride(0) if batched else 0
        if a.dtype == torch.float64 and M >= 64 and N >= 64 and K >= 16:
            _l.call("gb_gemm_f64", _l.ptr(a2), _l.ptr(b2), _l.ptr(out), _l.I(M), _l.I(N), _l.I(K), _l.I(batch),
                    _l.I(int(trans_a)), _l.I(int(trans_b)), _l.L(lda), _l.L(ldb), _l.L(out.stride(-2)), _l.L(sA),
                    _l.L(sB), _l.L(sC), _l.D(alpha), _l.I(int(beta)), _l.stream_ptr())
            return out
        if (a.dtype == torch.float32 and out.dtype == torch.float32 and _FP32_MODE == "bf16x3"
                and 2.0 * M * N * K * batch >= 2.0 ** 28 and M >= 128 and N >= 128
                and (K % 8 == 0 or (not trans_a and trans_b)) and out.stride(-2) % 4 == 0
                and out.data_ptr() % 16 == 0):
            need = int(_l.lib().gb_gemm_f32x3_workspace(M, N, K, batch))
            if need <= (4 << 30):
                ws3 = _x3_workspace(a.device, need)
                ws = _workspace(a.device) if M * N * batch * 4 * 2 <= _WS_BYTES else None
                _l.call("gb_gemm_f32x3", _l.ptr(a2), _l.ptr(b2), _l.ptr(out), _l.I(M), _l.I(N), _l.I(K),
                        _l.I(batch), _l.I(int(trans_a)), _l.I(int(trans_b)), _l.L(lda), _l.L(ldb),
                        _l.L(out.stride(-2)), _l.L(sA), _l.L(sB), _l.L(sC), _l.F(alpha), _l.I(int(beta)),
                        _l.ptr(ws3), _l.L(ws3.numel()), _l.ptr(ws), _l.L(_WS_BYTES if ws is not None else 0),
                        _l.stream_ptr())
                return out
        _l.call("gb_gemm_simt", _l.ptr(a2), _l.ptr(b2), _l.ptr(out), _l.I(M), _l.I(N), _l.I(K),
                _l.I(batch), _l.I(int(trans_a)), _l.I(int(trans_b)), _l.L(lda), _l.L(ldb),
                _l.L(out.stride(-2)), _l.L(sA), _l.L(sB), _l.L(sC), _l.I(_l.dtype_code(a.dtype)),
                _l.D(alpha), _l.I(int(beta)), _l.stream_ptr())
        return out

    # tensor-core path: contiguous dim pitch must be a multiple of 8 elements
    if (not batched and a.is_contiguous() and b.is_contiguous() and a.shape[1] % 8 == 0
            and b.shape[1] % 8 == 0 and a.data_ptr() % 16 == 0 and b.data_ptr() % 16 == 0):
        # the common case (two contiguous, aligned matrices): nothing to pad or copy
        a2, b2, lda, ldb, sA, sB = a, b, a.shape[1], b.shape[1], 0, 0
    else:
        a2 = _pad_last(a, 8)
        b2 = _pad_last(b, 8)
        a2, lda = _row_major_2d(a2)
        b2, ldb = _row_major_2d(b2)
        sA = a2.stride(0) if a2.dim() == 3 and a2.shape[0] > 1 else 0
        sB = b2.stride(0) if b2.dim() == 3 and b2.shape[0] > 1 else 0
    if batch > 1 and ((sA % 8) or (sB % 8)):
        a2 = a2.contiguous() if sA % 8 else a2
        b2 = b2.contiguous() if sB % 8 else b2
        if (a2.dim() == 3 and a2.stride(0) % 8) or (b2.dim() == 3 and b2.stride(0) % 8):
            raise ValueError("gemm: batch strides must be multiples of 8 elements")
        sA = a2.stride(0) if a2.dim() == 3 and a2.shape[0] > 1 else 0
        sB = b2.stride(0) if b2.dim() == 3 and b2.shape[0] > 1 else 0
    sC = out.stride(0) if batched else 0
    am = AUX[aux_mode] if aux is not None else 0
    if aux is not None:
        if aux.dtype != a.dtype or tuple(aux.shape) != oshape or aux.stride(-1) != 1:
            raise ValueError("gemm: aux must match the output shape and the input dtype")
    bias_f32 = 0
    if bias is not None:
        if bias.numel() != N:
            raise ValueError("gemm: bias must have N elements")
        if bias.dtype == torch.float32:
            bias_f32 = 1
        elif bias.dtype != a.dtype:
            bias = bias.to(torch.float32)
            bias_f32 = 1
        bias = bias.contiguous()
    if out.dtype not in (a.dtype, torch.float32):
        raise TypeError("gemm: out dtype must be the input dtype or float32")
    # split-K scratch: only products with a long K and few output tiles use it
    ws = None
    if K >= 2048 and bias is None and not ACT[act] and not am and M * N * batch * 4 * 2 <= _WS_BYTES:
        ws = _workspace(a.device)
    _l.call("gb_gemm16", _l.ptr(a2), _l.ptr(b2), _l.ptr(out), _l.ptr(bias), _l.I(bias_f32),
            _l.ptr(aux), _l.I(M), _l.I(N), _l.I(K), _l.I(batch), _l.I(int(trans_a)),
            _l.I(int(trans_b)), _l.L(lda), _l.L(ldb), _l.L(out.stride(-2)),
            _l.L(aux.stride(-2) if aux is not None else 0), _l.L(sA), _l.L(sB), _l.L(sC),
            _l.L(aux.stride(0) if (aux is not None and batched) else 0),
            _l.I(_l.dtype_code(a.dtype)), _l.I(_l.dtype_code(out.dtype)), _l.I(ACT[act]), _l.I(am),
            _l.I(int(beta)), _l.F(alpha), _l.I(force_bn), _l.ptr(ws), _l.L(_WS_BYTES if ws is not None else 0),
            _l.stream_ptr())
    return out


def _epilogue_torch(v, bias, act, aux, aux_mode, beta, out):
    if bias is not None:
        v = v + bias.to(v.dtype)
    m = AUX[aux_mode] if aux is not None else 0
    if m == 2:
        aux.copy_(v)
    v = _act_ref(v, act)
    if m == 1:
        v = v + aux
    elif m in (3, 4, 5):
        v = v * _dact_ref(aux, m)
    if beta:
        out.add_(v)
    else:
        out.copy_(v)
    return out

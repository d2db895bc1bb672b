"""Correctness check of the active compute backend against an independent reference.

    python -m gonn_b200.utils.verify            # CUDA backend when a device is present, else CPU
    python -m gonn_b200.utils.verify --device cpu

The counterpart of the reference's ``benchmark/verify`` program (benchmark/verify/main.go):
small inputs go through ``backend.Current()`` — every combination of batch size and
transposition flags of the GEMM contract, and every enum-dispatched unary and binary kind —
and are compared with formulas written here in numpy float64, which share no code with the
kernels or the oracle path.  On top of the reference's list the check covers the 16-bit
tensor-core GEMM, the multi-head-attention fast path against the materialised one, and the
device status word.  Prints one line per check and exits non-zero on the first mismatch.
"""
from __future__ import annotations

import argparse
import math
import sys
from typing import Callable, List

import numpy as np
import torch

from .. import backend as B


def ref_gemm(a: np.ndarray, b: np.ndarray, batch: int, m: int, k: int, n: int, trans_a: bool,
             trans_b: bool) -> np.ndarray:
    """Row-major batched ``op(A) @ op(B)`` on flat arrays: op(A) is stored (k, m) when
    ``trans_a``, op(B) is stored (n, k) when ``trans_b``."""
    A = a.reshape(batch, k, m).transpose(0, 2, 1) if trans_a else a.reshape(batch, m, k)
    Bm = b.reshape(batch, n, k).transpose(0, 2, 1) if trans_b else b.reshape(batch, k, n)
    return np.einsum("bik,bkj->bij", A, Bm).reshape(-1)


_erf = np.vectorize(math.erf)

REF_UNARY = {
    B.UnaryKind.ReLU: lambda x: np.maximum(x, 0.0),
    B.UnaryKind.Sigmoid: lambda x: 1.0 / (1.0 + np.exp(-x)),
    B.UnaryKind.Tanh: np.tanh,
    B.UnaryKind.Exp: np.exp,
    B.UnaryKind.Log: lambda x: np.log(np.abs(x) + 1.0),          # evaluated on |x| + 1
    B.UnaryKind.GELU: lambda x: 0.5 * x * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x ** 3))),
    B.UnaryKind.SiLU: lambda x: x / (1.0 + np.exp(-x)),
    B.UnaryKind.GELUExact: lambda x: 0.5 * x * (1.0 + _erf(x / math.sqrt(2.0))),
}
REF_BINARY = {
    B.BinaryKind.Add: np.add, B.BinaryKind.Sub: np.subtract, B.BinaryKind.Mul: np.multiply,
    B.BinaryKind.Div: np.divide,
}


class Report:
    def __init__(self, out=sys.stdout):
        self.out, self.failed = out, 0

    def check(self, label: str, got, want, tol: float) -> bool:
        got = np.asarray(got, dtype=np.float64).reshape(-1)
        want = np.asarray(want, dtype=np.float64).reshape(-1)
        diff = float(np.max(np.abs(got - want) / (1.0 + np.abs(want)))) if got.size else 0.0
        ok = got.shape == want.shape and math.isfinite(diff) and diff <= tol
        self.failed += 0 if ok else 1
        print(f"  {label:58s} maxRelDiff={diff:.3e}  [{'OK' if ok else 'FAIL'}]", file=self.out)
        return ok


def _np(t: torch.Tensor) -> np.ndarray:
    return t.detach().to("cpu", torch.float64).numpy()


def verify_gemm(rep: Report, dev: torch.device, dtype: torch.dtype, tol: float, rng) -> None:
    be = B.Current()
    for batch in (1, 3):
        for (m, k, n) in ((5, 7, 3), (16, 24, 8), (33, 40, 65)):
            if dtype in (torch.bfloat16, torch.float16) and (m, k, n) == (5, 7, 3):
                continue                                   # 16-bit pitches are multiples of 8
            for ta in (False, True):
                for tb in (False, True):
                    a = rng.standard_normal(batch * m * k)
                    b = rng.standard_normal(batch * k * n)
                    ta_t = torch.tensor(a, dtype=torch.float64).to(dev, dtype)
                    tb_t = torch.tensor(b, dtype=torch.float64).to(dev, dtype)
                    got = be.Gemm(ta_t, tb_t, batch, m, k, n, ta, tb)
                    want = ref_gemm(_np(ta_t), _np(tb_t), batch, m, k, n, ta, tb)
                    rep.check(f"gemm {str(dtype)[6:]} batch={batch} m={m} k={k} n={n} tA={int(ta)} tB={int(tb)}",
                              _np(got), want, tol)


def verify_elementwise(rep: Report, dev: torch.device, rng) -> None:
    be = B.Current()
    x = rng.standard_normal(1000) * 3.0
    y = rng.standard_normal(1000)
    y = np.where(np.abs(y) < 0.1, 0.5, y)
    for kind, f in REF_UNARY.items():
        xin = np.abs(x) + 1.0 if kind == B.UnaryKind.Log else x
        got = be.Unary(kind, torch.tensor(xin, dtype=torch.float64, device=dev))
        want = np.log(xin) if kind == B.UnaryKind.Log else f(x)
        rep.check(f"unary {kind.name}", _np(got), want, 1e-12)
    for kind, f in REF_BINARY.items():
        got = be.Binary(kind, torch.tensor(x, dtype=torch.float64, device=dev),
                        torch.tensor(y, dtype=torch.float64, device=dev))
        rep.check(f"binary {kind.name}", _np(got), f(x, y), 1e-12)


def verify_attention(rep: Report, dev: torch.device, rng) -> None:
    """``MultiHeadAttention.ForwardFused`` against the materialised path (benchmark/mha/main.go:55-73) and
    against softmax attention written out in numpy."""
    from .. import nn
    torch.manual_seed(0)
    E, H, Bsz, S = 128, 2, 2, 48
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float64
    tol = 3e-2 if dev.type == "cuda" else 1e-9
    mtol = 3e-2 if dev.type == "cuda" else 1e-5
    mha = nn.MultiHeadAttention(E, H).to(device=dev, dtype=dtype)
    x = torch.tensor(rng.standard_normal((Bsz, S, E)), dtype=torch.float64).to(dev, dtype)
    for causal in (False, True):
        with torch.no_grad():
            ref = mha.ForwardMasked(x, x, x, causal)     # materialised (S, S) scores, fp32
            fused = mha.ForwardFused(x, x, x, causal)
        rep.check(f"MultiHeadAttention fused vs materialised causal={causal}", _np(fused), _np(ref), mtol)
    # the attention core alone, in numpy
    from ..ops.attention import flash_attention
    D = 64
    q, k, v = (torch.tensor(rng.standard_normal((1, S, 2, D)), dtype=torch.float64).to(dev, dtype) for _ in range(3))
    for causal in (False, True):
        got = flash_attention(q, k, v, causal)
        qn, kn, vn = (_np(t).transpose(0, 2, 1, 3) for t in (q, k, v))
        s = np.einsum("bhid,bhjd->bhij", qn, kn) / math.sqrt(D)
        if causal:
            s = np.where(np.triu(np.ones((S, S), dtype=bool), 1), -np.inf, s)
        p = np.exp(s - s.max(-1, keepdims=True))
        p /= p.sum(-1, keepdims=True)
        want = np.einsum("bhij,bhjd->bhid", p, vn).transpose(0, 2, 1, 3)
        rep.check(f"attention core causal={causal}", _np(got), want, tol)


def verify_attention_backward(rep: Report, dev: torch.device, rng) -> None:
    """The reference's backward check (benchmark/flashbwd/main.go:41-139): central differences of
    ``sum(O * dO)`` (eps 1e-6, float64) against the analytic dQ, dK and dV at six positions, (BH, S, D) =
    (2, 6, 64), causal and not, relative error below 1e-4; then a one-head attention layer of width 64
    trained for 30 Adam steps on a fixed target must lower its squared error."""
    from .. import nn, optim
    from ..ops.attention import flash_attention
    BH, S, D = 2, 6, 64
    n = BH * S * D
    for causal in (False, True):
        q, k, v, do = (torch.tensor(rng.standard_normal((1, S, BH, D)), dtype=torch.float64, device=dev) for _ in range(4))
        leaves = [t.clone().requires_grad_(True) for t in (q, k, v)]
        flash_attention(*leaves, causal).backward(do)

        def loss(ts):
            with torch.no_grad():
                return float((flash_attention(*ts, causal) * do).sum())

        got, want = [], []
        for which in range(3):
            for idx in (0, 1, 64, 130, 200, n - 1):
                ts = [q.clone(), k.clone(), v.clone()]
                flat = ts[which].view(-1)
                x0 = float(flat[idx])
                flat[idx] = x0 + 1e-6
                lp = loss(ts)
                flat[idx] = x0 - 1e-6
                lm = loss(ts)
                want.append((lp - lm) / 2e-6)
                got.append(float(leaves[which].grad.reshape(-1)[idx]))
        rep.check(f"attention backward vs central differences causal={causal}", got, want, 1e-4)
    torch.manual_seed(1)
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float64
    mha = nn.MultiHeadAttention(64, 1).to(device=dev, dtype=dtype)
    opt = optim.Adam(mha.parameters(), lr=1e-2)
    x = torch.tensor(rng.standard_normal((2, 8, 64)), dtype=torch.float64).to(dev, dtype)
    target = torch.tensor(rng.standard_normal((2, 8, 64)), dtype=torch.float64).to(dev, dtype)
    first = last = 0.0
    for step in range(30):
        opt.zero_grad()
        err = mha(x, x, x, True) - target
        l = (err * err).mean()
        l.backward()
        opt.step()
        last = float(l.detach())
        first = last if step == 0 else first
    ok = last < first
    rep.failed += 0 if ok else 1
    print(f"  {'attention layer training, 30 Adam steps':58s} loss {first:.5f} -> {last:.5f}  [{'OK' if ok else 'FAIL'}]",
          file=rep.out)


def run(device: str, out=sys.stdout) -> int:
    dev = torch.device(device)
    prev = B.Use(B.NewCUDA() if dev.type == "cuda" else B.NewCPU())
    rep = Report(out)
    rng = np.random.default_rng(1234)
    try:
        print(f"backend: {B.Current().Name()}", file=out)
        verify_gemm(rep, dev, torch.float64, 1e-11, rng)
        verify_gemm(rep, dev, torch.float32, 2e-5, rng)
        if dev.type == "cuda":
            verify_gemm(rep, dev, torch.bfloat16, 2e-2, rng)
            verify_gemm(rep, dev, torch.float16, 4e-3, rng)
        verify_elementwise(rep, dev, rng)
        verify_attention(rep, dev, rng)
        verify_attention_backward(rep, dev, rng)
        if dev.type == "cuda":
            from .. import lib
            B.Current().Synchronize()
            code = lib.read_status()[0]
            rep.check("device status word", [code], [0], 0.0)
    finally:
        B.Use(prev)
    print("ALL CHECKS PASSED" if rep.failed == 0 else f"{rep.failed} CHECKS FAILED", file=out)
    return 1 if rep.failed else 0


def main(argv: List[str]) -> int:
    ap = argparse.ArgumentParser(prog="verify")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    return run(ap.parse_args(argv).device)


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))

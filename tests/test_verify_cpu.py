"""The backend verification program: passes on the CPU backend, flags a wrong backend."""
import io

import numpy as np
import torch

from gonn_b200 import backend as B
from gonn_b200.utils import verify as V


def test_verify_passes_on_cpu_backend():
    out = io.StringIO()
    assert V.run("cpu", out) == 0
    text = out.getvalue()
    assert "ALL CHECKS PASSED" in text and "FAIL" not in text.replace("FAILED", "")
    assert text.count("gemm float64") == 2 * 3 * 4 and "unary GELUExact" in text and "binary Div" in text
    assert text.count("attention backward vs central differences") == 2
    assert "attention layer training, 30 Adam steps" in text


def test_verify_flags_a_backend_that_ignores_transposition():
    class Wrong(B.NativeBackend):
        def Gemm(self, a, b, batch, m, k, n, transA=False, transB=False):
            if transA:                       # reads op(A) as if it were stored (m, k)
                return torch.bmm(a.reshape(batch, m, k), (b.reshape(batch, n, k).transpose(1, 2) if transB
                                                           else b.reshape(batch, k, n)))
            return super().Gemm(a, b, batch, m, k, n, transA, transB)

    prev = B.Use(Wrong("cpu"))
    try:
        rep = V.Report(io.StringIO())
        V.verify_gemm(rep, torch.device("cpu"), torch.float64, 1e-11, np.random.default_rng(0))
    finally:
        B.Use(prev)
    assert rep.failed == 2 * 3 * 2          # every transA case, none of the others


def test_reference_gemm_against_loops():
    rng = np.random.default_rng(3)
    batch, m, k, n = 2, 3, 4, 5
    a, b = rng.standard_normal(batch * m * k), rng.standard_normal(batch * k * n)
    for ta in (False, True):
        for tb in (False, True):
            want = np.zeros(batch * m * n)
            for bi in range(batch):
                for i in range(m):
                    for j in range(n):
                        s = 0.0
                        for p in range(k):
                            av = a[bi * m * k + (p * m + i if ta else i * k + p)]
                            bv = b[bi * k * n + (j * k + p if tb else p * n + j)]
                            s += av * bv
                        want[(bi * m + i) * n + j] = s
            np.testing.assert_allclose(V.ref_gemm(a, b, batch, m, k, n, ta, tb), want, rtol=1e-13)

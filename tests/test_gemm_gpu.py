"""tcgen05 GEMM against an fp32 torch reference: all trans layouts, ragged shapes,
batched, epilogues.  (Pattern: benchmark/verify/main.go:77-201 of the reference checks
GEMM NN/TN/NT/TT/batched against a naive reference.)"""
import pytest
import torch

from gonn_b200.ops.gemm import gemm

pytestmark = pytest.mark.gpu


def _ref(a, b, ta, tb):
    A = a.float().transpose(-1, -2) if ta else a.float()
    B = b.float().transpose(-1, -2) if tb else b.float()
    return A @ B


def _mk(M, N, K, ta, tb, batch=0, dtype=torch.bfloat16):
    sa = (K, M) if ta else (M, K)
    sb = (N, K) if tb else (K, N)
    if batch:
        sa, sb = (batch,) + sa, (batch,) + sb
    return (torch.randn(sa, device="cuda", dtype=dtype), torch.randn(sb, device="cuda", dtype=dtype))


@pytest.mark.parametrize("ta", [False, True])
@pytest.mark.parametrize("tb", [False, True])
@pytest.mark.parametrize("shape", [(256, 512, 256), (200, 136, 72), (128, 128, 64), (1000, 24, 520)])
@pytest.mark.parametrize("bn", [0, 128, 256])
def test_layouts(ta, tb, shape, bn, status_ok):
    M, N, K = shape
    a, b = _mk(M, N, K, ta, tb)
    c = gemm(a, b, trans_a=ta, trans_b=tb, force_bn=bn)
    ref = _ref(a, b, ta, tb)
    _close16(c, ref)


def _close16(c, ref):
    """A 16-bit result of an fp32 accumulation: every element within one rounding step of its
    own magnitude (2^-8 relative for bf16) plus the fp32 accumulation error of the row."""
    assert ((c.float() - ref).abs() <= 2.0 ** -8 * ref.abs() + 2e-3).all(), \
        float(((c.float() - ref).abs() - 2.0 ** -8 * ref.abs()).max())


@pytest.mark.parametrize("ta,tb", [(False, True), (False, False), (True, False)])
def test_batched(ta, tb, status_ok):
    a, b = _mk(192, 160, 96, ta, tb, batch=5)
    c = gemm(a, b, trans_a=ta, trans_b=tb)
    ref = _ref(a, b, ta, tb)
    _close16(c, ref)


def test_batch_broadcast(status_ok):
    a = torch.randn(4, 128, 64, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(64, 96, device="cuda", dtype=torch.bfloat16)
    c = gemm(a, b)
    ref = a.float() @ b.float()
    _close16(c, ref)


@pytest.mark.parametrize("ta", [False, True])
@pytest.mark.parametrize("tb", [False, True])
@pytest.mark.parametrize("shape", [(256, 256, 256), (200, 136, 72), (129, 65, 17), (1000, 64, 520)])
def test_fp64_tensor_core_gemm(ta, tb, shape, status_ok):
    """The double-precision tensor-core kernel against torch's float64 product: agreement at
    the level of float64 summation-order differences, all layouts, ragged edges."""
    M, N, K = shape
    a, b = _mk(M, N, K, ta, tb, dtype=torch.float64)
    c = gemm(a, b, trans_a=ta, trans_b=tb)
    A = a.transpose(-1, -2) if ta else a
    B = b.transpose(-1, -2) if tb else b
    ref = A @ B
    assert c.dtype == torch.float64
    assert (c - ref).abs().max().item() < 1e-12 * (K ** 0.5) * (1 + ref.abs().max().item())


def test_fp64_tensor_core_batched_alpha_beta(status_ok):
    a, b = _mk(192, 160, 96, False, True, batch=3, dtype=torch.float64)
    out = torch.randn(3, 192, 160, device="cuda", dtype=torch.float64)
    want = out + 0.5 * (a @ b.transpose(-1, -2))
    gemm(a, b, trans_b=True, out=out, beta=True, alpha=0.5)
    assert (out - want).abs().max().item() < 1e-11
    # a broadcast right operand
    b1 = torch.randn(96, 160, device="cuda", dtype=torch.float64)
    c = gemm(a, b1)
    assert (c - a @ b1).abs().max().item() < 1e-11


@pytest.mark.parametrize("ta,tb", [(False, True), (False, False), (True, False), (True, True)])
@pytest.mark.parametrize("shape", [(1024, 1024, 1024), (640, 520, 1000)])
def test_fp32_three_plane_gemm(ta, tb, shape, status_ok):
    """fp32 products on the tensor cores (three bf16 planes per operand): against float64 math the
    error must stay at the level of an fp32 FMA chain, measured against the same chain in torch."""
    from gonn_b200.ops.gemm import set_fp32_gemm_mode
    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(M + K)
    sa = (K, M) if ta else (M, K)
    sb = (N, K) if tb else (K, N)
    a = torch.randn(sa, device="cuda", generator=g) * torch.exp(torch.randn(sa, device="cuda", generator=g))
    b = torch.randn(sb, device="cuda", generator=g)
    A = a.transpose(-1, -2) if ta else a
    B = b.transpose(-1, -2) if tb else b
    ref = A.double() @ B.double()
    scale = (A.double().abs() @ B.double().abs())           # size of the terms that were summed
    old = set_fp32_gemm_mode("bf16x3")
    try:
        c = gemm(a, b, trans_a=ta, trans_b=tb)
        set_fp32_gemm_mode("simt")
        c_simt = gemm(a, b, trans_a=ta, trans_b=tb)
    finally:
        set_fp32_gemm_mode(old)
    err = ((c.double() - ref).abs() / scale).max().item()
    err_simt = ((c_simt.double() - ref).abs() / scale).max().item()
    assert c.dtype == torch.float32
    # both within a few units of 2^-24 of the summed magnitude (the three passes by magnitude
    # class are what keeps the plane scheme there: one pass over all six products loses the low planes)
    assert err < 1e-6, (err, err_simt)
    assert err_simt < 1e-6, err_simt


def test_fp32_three_plane_alpha_beta_batched_nonfinite(status_ok):
    a = torch.randn(2, 512, 512, device="cuda")
    b = torch.randn(2, 512, 512, device="cuda")
    out = torch.randn(2, 512, 512, device="cuda")
    want = out.double() + 2.0 * (a.double() @ b.double().transpose(-1, -2))
    gemm(a, b, trans_b=True, out=out, beta=True, alpha=2.0)
    assert (out.double() - want).abs().max().item() < 2e-4
    a2 = torch.randn(512, 1024, device="cuda")
    b2 = torch.randn(1024, 512, device="cuda")
    a2[3, 5] = float("inf")
    c = gemm(a2, b2)
    row = c[3]
    assert torch.isinf(row).all() or torch.isnan(row).any()          # the infinite entry stays visible
    ok = torch.ones(512, dtype=torch.bool, device="cuda")
    ok[3] = False
    assert torch.isfinite(c[ok]).all()


def test_fp16_and_fp32_out(status_ok):
    a, b = _mk(256, 256, 256, False, True, dtype=torch.float16)
    c = gemm(a, b, trans_b=True, out_dtype=torch.float32)
    ref = _ref(a, b, False, True)
    assert c.dtype == torch.float32
    assert (c - ref).abs().max().item() < 1e-2


def test_unaligned_inner_dims(status_ok):
    # N = 10 and K = 27 are not multiples of 8: the wrapper pads the pitch
    a = torch.randn(64, 27, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(10, 27, device="cuda", dtype=torch.bfloat16)
    c = gemm(a, w, trans_b=True)
    ref = a.float() @ w.float().T
    assert c.shape == (64, 10)
    assert (c.float() - ref).abs().max().item() < 0.2
    dy = torch.randn(64, 10, device="cuda", dtype=torch.bfloat16)
    dx = gemm(dy, w)
    assert (dx.float() - dy.float() @ w.float()).abs().max().item() < 0.2
    dw = gemm(dy, a, trans_a=True)
    assert (dw.float() - dy.float().T @ a.float()).abs().max().item() < 0.5


@pytest.mark.parametrize("act", [None, "relu", "gelu", "geluexact"])
def test_bias_activation_epilogue(act, status_ok):
    M, N, K = 384, 520, 256
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    pre = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    y = gemm(a, w, trans_b=True, bias=bias, act=act, aux=pre, aux_mode="store_pre")
    rp = a.float() @ w.float().T + bias.float()
    F = torch.nn.functional
    ry = {None: rp, "relu": torch.relu(rp), "gelu": F.gelu(rp, approximate="tanh"), "geluexact": F.gelu(rp)}[act]
    assert (pre.float() - rp).abs().max().item() < 0.03
    assert (y.float() - ry).abs().max().item() < 0.03


def test_residual_and_dact_epilogues(status_ok):
    M, N, K = 256, 256, 128
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
    res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    y = gemm(a, w, trans_b=True, aux=res, aux_mode="add")
    ref = a.float() @ w.float().T + res.float()
    assert (y.float() - ref).abs().max().item() < 0.05
    pre = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    y2 = gemm(a, w, trans_b=True, aux=pre, aux_mode="mul_dgelu")
    p = pre.float().requires_grad_(True)
    torch.nn.functional.gelu(p, approximate="tanh").sum().backward()
    ref2 = (a.float() @ w.float().T) * p.grad
    assert (y2.float() - ref2).abs().max().item() < 0.05


def test_beta_accumulate(status_ok):
    a, b = _mk(128, 256, 64, False, True)
    out = torch.ones(128, 256, device="cuda", dtype=torch.float32)
    gemm(a, b, trans_b=True, out=out, beta=True)
    ref = _ref(a, b, False, True) + 1
    assert (out - ref).abs().max().item() < 1e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_simt_exact(dtype, status_ok):
    a = torch.randn(70, 50, device="cuda", dtype=dtype)
    b = torch.randn(50, 33, device="cuda", dtype=dtype)
    c = gemm(a, b)
    tol = 1e-10 if dtype == torch.float64 else 1e-4
    assert (c - a @ b).abs().max().item() < tol
    c2 = gemm(a, b.t().contiguous(), trans_b=True)
    assert (c2 - a @ b).abs().max().item() < tol
    c3 = gemm(a.t().contiguous(), b, trans_a=True)
    assert (c3 - a @ b).abs().max().item() < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_simt_tiled_large_ragged_batched(dtype, status_ok):
    """Enough tiles for the 128-row configuration, ragged edges, every transposition, batch
    strides, accumulation onto the output and a scaled product."""
    tol = 1e-9 if dtype == torch.float64 else 2e-3
    M, N, K = 1300, 1501, 70
    a = torch.randn(M, K, device="cuda", dtype=dtype)
    b = torch.randn(K, N, device="cuda", dtype=dtype)
    ref = a.double() @ b.double()
    for ta in (False, True):
        for tb in (False, True):
            aa = a.t().contiguous() if ta else a
            bb = b.t().contiguous() if tb else b
            c = gemm(aa, bb, trans_a=ta, trans_b=tb)
            assert (c.double() - ref).abs().max().item() < tol, (ta, tb)
    out = torch.ones(M, N, device="cuda", dtype=dtype)
    gemm(a, b, out=out, beta=True, alpha=0.5)
    assert (out.double() - (0.5 * ref + 1)).abs().max().item() < tol
    a3 = torch.randn(5, 200, 96, device="cuda", dtype=dtype)
    b3 = torch.randn(5, 96, 330, device="cuda", dtype=dtype)
    assert (gemm(a3, b3).double() - torch.bmm(a3.double(), b3.double())).abs().max().item() < tol
    assert (gemm(a3, b3[0]).double() - torch.matmul(a3.double(), b3[0].double())).abs().max().item() < tol


def test_large_matches_reference(status_ok):
    a, b = _mk(2048, 2048, 2048, False, True)
    c = gemm(a, b, trans_b=True)
    ref = _ref(a, b, False, True)
    assert (c.float() - ref).abs().max().item() < 0.01 * ref.abs().max().item() + 0.1

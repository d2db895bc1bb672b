"""Memory-bound kernels (elementwise, norms, softmax / cross-entropy, embedding,
reductions, optimizers, dropout) against fp32 / fp64 torch references on the GPU.
Pattern: tensor/cuda_dispatch_test.go of the reference (GPU vs host at tight tolerance)."""
import math

import pytest
import torch

from gonn_b200.ops import elementwise as ew
from gonn_b200.ops.embedding import embedding
from gonn_b200.ops.norm import layer_norm, norm_ref, rms_norm
from gonn_b200.ops.reduce import reduce_axis
from gonn_b200.ops.softmax import cross_entropy, cross_entropy_ref, log_softmax, softmax

pytestmark = pytest.mark.gpu
F = torch.nn.functional

_POS = {"log", "sqrt", "reciprocal", "pow"}
_PARAMS = {"pow": (2.5, 0), "clip": (-0.5, 0.7), "leakyrelu": (0.1, 0), "elu": (1.3, 0), "hardshrink": (0.4, 0),
           "softshrink": (0.4, 0), "softplusbeta": (2.0, 10.0), "threshold": (0.2, -1.0), "celu": (1.5, 0),
           "scale_add": (1.5, -0.25)}


@pytest.mark.parametrize("name", sorted(ew.UNARY_IDS))
@pytest.mark.parametrize("dtype", [torch.float64, torch.float32, torch.bfloat16])
def test_unary_forward_backward(name, dtype, status_ok):
    n = 10007
    x = torch.randn(n, device="cuda", dtype=torch.float64) * 2
    if name in _POS:
        x = x.abs() + 0.1
    if name == "tan":
        x = x.clamp(-1.2, 1.2)
    x = x.to(dtype)
    p0, p1 = _PARAMS.get(name, (0.0, 0.0))
    y = ew.unary_forward(name, x, p0, p1)
    fwd, bwd = ew._REF[name]
    xr = x.double()
    tol = {torch.float64: 1e-9, torch.float32: 2e-4, torch.bfloat16: 3e-2}[dtype]
    ref = fwd(xr, p0, p1)
    assert ((y.double() - ref).abs() / (1 + ref.abs())).max().item() < tol
    dy = torch.randn(n, device="cuda", dtype=torch.float64).to(dtype)
    dx = ew.unary_backward(name, x, dy, p0, p1)
    refd = dy.double() * bwd(xr, p0, p1)
    assert ((dx.double() - refd).abs() / (1 + refd.abs())).max().item() < tol


def test_registry_has_25_names():
    assert len(ew.REGISTERED_UNARY) == 25


@pytest.mark.parametrize("name", ["add", "sub", "mul", "div"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float64])
def test_binary_broadcast_and_grad(name, dtype, status_ok):
    a = torch.randn(4, 1, 33, device="cuda", dtype=dtype).requires_grad_(True)
    b = (torch.randn(5, 33, device="cuda", dtype=dtype).abs() + 0.5).requires_grad_(True)
    y = ew.binary(name, a, b)
    ref = getattr(torch, name)(a.detach().double(), b.detach().double())
    tol = {torch.float64: 1e-12, torch.float32: 1e-5, torch.bfloat16: 5e-2}[dtype]
    assert y.shape == ref.shape
    assert (y.double() - ref).abs().max().item() < tol * (1 + ref.abs().max().item())
    g = torch.randn_like(y)
    y.backward(g)
    ad, bd = a.detach().double().requires_grad_(True), b.detach().double().requires_grad_(True)
    getattr(torch, name)(ad, bd).backward(g.double())
    assert (a.grad.double() - ad.grad).abs().max().item() < 20 * tol * (1 + ad.grad.abs().max().item())
    assert (b.grad.double() - bd.grad).abs().max().item() < 20 * tol * (1 + bd.grad.abs().max().item())


@pytest.mark.parametrize("name", ["add", "sub", "mul", "div"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float64])
@pytest.mark.parametrize("shapes", [((37, 64), (64,)), ((3, 5, 48), (1, 5, 48)), ((64,), (9, 64)), ((1, 7, 16), (4, 7, 16)),
                                    ((6, 40), (40,)), ((2, 3, 4, 8), (4, 8)), ((5, 12), (12,))])
def test_binary_row_vector_broadcast(name, dtype, shapes, status_ok):
    """One operand covers the whole output, the other repeats along the leading dimensions: the vectorised
    kernel when the repeating block is a whole number of 16-byte vectors (either side; the order matters for
    sub / div), the general kernel otherwise — same results."""
    sa, sb = shapes
    a = torch.randn(*sa, device="cuda").to(dtype)
    b = (torch.randn(*sb, device="cuda").abs() + 0.5).to(dtype)
    y = ew.binary_forward(name, a, b)
    ref = getattr(torch, name)(a.double(), b.double())
    tol = {torch.float64: 1e-12, torch.float32: 1e-5, torch.bfloat16: 5e-2}[dtype]
    assert y.shape == ref.shape
    assert (y.double() - ref).abs().max().item() < tol * (1 + ref.abs().max().item())


@pytest.mark.parametrize("op", ["argmax", "argmin"])
@pytest.mark.parametrize("shape,axis", [((1000, 70), 0), ((3, 257, 33), 1), ((64, 5), 0), ((2, 4096, 8), 1)])
def test_arg_reduction_over_an_inner_axis(op, shape, axis, status_ok):
    from gonn_b200.ops.reduce import reduce_axis
    x = torch.randn(*shape, device="cuda").to(torch.bfloat16)       # 16-bit values: ties are common
    got = reduce_axis(x, axis, op)
    # the first occurrence wins, as in a serial scan
    xf = x.float()
    ext = xf.max(axis, keepdim=True).values if op == "argmax" else xf.min(axis, keepdim=True).values
    idx = torch.arange(shape[axis], device="cuda").view([-1 if i == axis else 1 for i in range(len(shape))])
    want = torch.where(xf == ext, idx, shape[axis]).min(axis).values
    assert torch.equal(got.long(), want)


@pytest.mark.parametrize("D", [64, 768, 1000, 2048, 4096, 50])
@pytest.mark.parametrize("dtype,wdtype", [(torch.bfloat16, torch.bfloat16), (torch.float32, torch.float32),
                                          (torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("rms", [False, True])
def test_norms(D, dtype, wdtype, rms, status_ok):
    rows = 300
    x = torch.randn(rows, D, device="cuda", dtype=dtype).requires_grad_(True)
    w = (torch.randn(D, device="cuda") * 0.5 + 1).to(wdtype).requires_grad_(True)
    b = None if rms else torch.randn(D, device="cuda").to(wdtype).requires_grad_(True)
    y = rms_norm(x, w, 1e-6) if rms else layer_norm(x, w, b, 1e-5)
    xr, wr = x.detach().double().requires_grad_(True), w.detach().double().requires_grad_(True)
    br = None if rms else b.detach().double().requires_grad_(True)
    ref = norm_ref(xr, wr, br, 1e-6 if rms else 1e-5, rms)
    tol = 3e-2 if dtype == torch.bfloat16 else 1e-4
    assert ((y.double() - ref).abs() / (1 + ref.abs())).max().item() < tol
    g = torch.randn_like(y)
    y.backward(g)
    ref.backward(g.double())
    assert ((x.grad.double() - xr.grad).abs() / (1 + xr.grad.abs())).max().item() < tol * 3
    wt = 0.5 if wdtype == torch.bfloat16 else (0.15 if dtype == torch.bfloat16 else 1e-3)
    assert (w.grad.double() - wr.grad).abs().max().item() < wt * (1 + wr.grad.abs().max().item() * 0.05)
    if not rms:
        assert (b.grad.double() - br.grad).abs().max().item() < wt * (1 + br.grad.abs().max().item() * 0.05)


@pytest.mark.parametrize("pipelined", [1, 0])
@pytest.mark.parametrize("rows,D", [(1, 768), (7, 256), (300, 512), (4099, 768), (1030, 1024), (515, 1536),
                                    (300, 2048), (130, 3072), (70, 4096), (33, 6144), (20, 8192)])
@pytest.mark.parametrize("rms", [False, True])
def test_norm_kernels_tight(rows, D, rms, pipelined, status_ok):
    """bf16 rows with fp32 weights against float64 math: the output within one bf16 rounding
    step, the parameter gradients (fp32, deterministic fixed-order sums) to 1e-3 of their
    scale; every row-width class of the pipelined and of the register-resident kernels, with
    row counts that leave a ragged last tile."""
    from gonn_b200 import lib as gl
    gl.call("gb_norm_tune", gl.I(pipelined))
    try:
        g = torch.Generator(device="cuda").manual_seed(rows * 31 + D)
        x = (torch.randn(rows, D, device="cuda", generator=g) * 2 + 0.5).to(torch.bfloat16).requires_grad_(True)
        w = (torch.randn(D, device="cuda", generator=g) * 0.5 + 1).requires_grad_(True)
        b = None if rms else torch.randn(D, device="cuda", generator=g).requires_grad_(True)
        y = rms_norm(x, w, 1e-6) if rms else layer_norm(x, w, b, 1e-5)
        xr, wr = x.detach().double().requires_grad_(True), w.detach().double().requires_grad_(True)
        br = None if rms else b.detach().double().requires_grad_(True)
        ref = norm_ref(xr, wr, br, 1e-6 if rms else 1e-5, rms)
        assert ((y.double() - ref).abs() / (1 + ref.abs())).max().item() < 2 ** -8
        dy = torch.randn(rows, D, device="cuda", generator=g).to(torch.bfloat16)
        y.backward(dy)
        ref.backward(dy.double())
        assert ((x.grad.double() - xr.grad).abs() / (1 + xr.grad.abs())).max().item() < 2 ** -7
        scale = wr.grad.abs().max().item() + 1
        assert (w.grad.double() - wr.grad).abs().max().item() < 1e-3 * scale
        if not rms:
            assert (b.grad.double() - br.grad).abs().max().item() < 1e-3 * (br.grad.abs().max().item() + 1)
        # run to run: identical bytes
        x2 = x.detach().clone().requires_grad_(True)
        w2 = w.detach().clone().requires_grad_(True)
        b2 = None if rms else b.detach().clone().requires_grad_(True)
        y2 = rms_norm(x2, w2, 1e-6) if rms else layer_norm(x2, w2, b2, 1e-5)
        y2.backward(dy)
        assert torch.equal(y2, y) and torch.equal(x2.grad, x.grad) and torch.equal(w2.grad, w.grad)
    finally:
        gl.call("gb_norm_tune", gl.I(1))


@pytest.mark.parametrize("rows,D", [(5, 64), (300, 512), (4099, 768), (1030, 1024), (300, 2048), (70, 4096),
                                    (20, 8192)])
@pytest.mark.parametrize("rms", [False, True])
@pytest.mark.parametrize("wdtype", [torch.bfloat16, torch.float32])
def test_norm_fork_backward(rows, D, rms, wdtype, status_ok):
    """``norm_fork`` returns (norm(x), x); its one-kernel backward must equal norm_bwd(dy) + dpass,
    with the column sums of dpass as the gradient of ``res_bias`` (float64 reference)."""
    from gonn_b200.ops.norm import norm_fork
    g = torch.Generator(device="cuda").manual_seed(rows + D)
    x = (torch.randn(rows, D, device="cuda", generator=g) * 1.5).to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(D, device="cuda", generator=g) * 0.5 + 1).to(wdtype).requires_grad_(True)
    b = None if rms else torch.randn(D, device="cuda", generator=g).to(wdtype).requires_grad_(True)
    rb = torch.zeros(D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y, xp = norm_fork(x, w, b, 1e-5, rms, rb)
    assert torch.equal(xp, x)
    dy = torch.randn(rows, D, device="cuda", generator=g).to(torch.bfloat16)
    dp = torch.randn(rows, D, device="cuda", generator=g).to(torch.bfloat16)
    torch.autograd.backward([y, xp], [dy, dp])
    xr, wr = x.detach().double().requires_grad_(True), w.detach().double().requires_grad_(True)
    br = None if rms else b.detach().double().requires_grad_(True)
    ref = norm_ref(xr, wr, br, 1e-5, rms)
    ref.backward(dy.double())
    want_dx = xr.grad + dp.double()
    assert ((y.double() - ref).abs() / (1 + ref.abs())).max().item() < 2 ** -7
    assert ((x.grad.double() - want_dx).abs() / (1 + want_dx.abs())).max().item() < 2 ** -6
    wtol = 1e-3 if wdtype == torch.float32 else 2 ** -7
    assert (w.grad.double() - wr.grad).abs().max().item() < wtol * (wr.grad.abs().max().item() + 1)
    if not rms:
        assert (b.grad.double() - br.grad).abs().max().item() < wtol * (br.grad.abs().max().item() + 1)
    want_rb = dp.double().sum(0)
    assert (rb.grad.double() - want_rb).abs().max().item() < 2 ** -7 * (want_rb.abs().max().item() + 1)


@pytest.mark.parametrize("D", [10, 1000, 32000, 50304])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_softmax_family(D, dtype, status_ok):
    x = (torch.randn(37, D, device="cuda") * 3).to(dtype).requires_grad_(True)
    for fn, tfn in ((softmax, torch.softmax), (log_softmax, torch.log_softmax)):
        x.grad = None
        y = fn(x, -1)
        xr = x.detach().double().requires_grad_(True)
        ref = tfn(xr, -1)
        tol = 3e-2 if dtype == torch.bfloat16 else 1e-5
        assert (y.double() - ref).abs().max().item() < tol * (1 + ref.abs().max().item() * 0.1)
        g = torch.randn_like(y)
        y.backward(g)
        ref.backward(g.double())
        assert (x.grad.double() - xr.grad).abs().max().item() < tol * (1 + xr.grad.abs().max().item())


def test_softmax_other_axis(status_ok):
    x = torch.randn(4, 7, 9, device="cuda")
    assert (softmax(x, 1) - torch.softmax(x, 1)).abs().max().item() < 1e-6


@pytest.mark.parametrize("C", [10, 1000, 32000])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("opts", [dict(), dict(ignore_index=3), dict(label_smoothing=0.1), dict(weighted=True),
                                  dict(weighted=True, label_smoothing=0.2, ignore_index=1), dict(reduction="sum"),
                                  dict(reduction="none")])
def test_cross_entropy(C, dtype, opts, status_ok):
    opts = dict(opts)
    N = 129
    x = (torch.randn(N, C, device="cuda") * 2).to(dtype).requires_grad_(True)
    t = torch.randint(0, C, (N,), device="cuda")
    t[:5] = torch.tensor([3, 1, 3, 1, 0], device="cuda")
    w = (torch.rand(C, device="cuda") + 0.5) if opts.pop("weighted", False) else None
    loss = cross_entropy(x, t, weight=w, **opts)
    xr = x.detach().double().requires_grad_(True)
    ref = cross_entropy_ref(xr, t, weight=w, **opts)
    tl = F.cross_entropy(xr.detach(), t, weight=None if w is None else w.double(),
                         ignore_index=opts.get("ignore_index", -100),
                         label_smoothing=opts.get("label_smoothing", 0.0),
                         reduction=opts.get("reduction", "mean"))
    assert (ref.detach() - tl).abs().max().item() < 1e-9  # the oracle equals torch's semantics
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    assert (loss.double() - ref.detach()).abs().max().item() < tol * (1 + ref.abs().max().item())
    g = torch.randn_like(loss) if loss.dim() else torch.tensor(1.7, device="cuda")
    loss.backward(g)
    ref.backward(g.double())
    assert (x.grad.double() - xr.grad).abs().max().item() < tol * (0.02 + xr.grad.abs().max().item())


def test_cross_entropy_inplace_backward(status_ok):
    x = torch.randn(64, 500, device="cuda", dtype=torch.bfloat16)
    t = torch.randint(0, 500, (64,), device="cuda")
    lin = torch.nn.Parameter(x.clone())
    logits = lin * 1.0
    loss = cross_entropy(logits, t, inplace_backward=True)
    loss.backward()
    xr = x.double().requires_grad_(True)
    F.cross_entropy(xr, t).backward()
    assert (lin.grad.double() - xr.grad).abs().max().item() < 1e-3


@pytest.mark.parametrize("N,C", [(64, 512), (257, 32000), (5, 8), (100, 1000)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("reduction,upstream", [("mean", 1.0), ("mean", 0.25), ("sum", 1.0)])
def test_cross_entropy_that_consumes_the_logits(N, C, dtype, reduction, upstream, status_ok):
    """One kernel for loss and gradient: the loss matches, the gradient that reaches the producer of the
    logits matches (also when the loss is scaled before backward), and the logits buffer holds it."""
    x = (torch.randn(N, C, device="cuda") * 2).to(dtype)
    t = torch.randint(0, C, (N,), device="cuda")
    src = torch.nn.Parameter(x.clone())
    logits = src * 1.0                                   # a non-leaf, as a model's head output is
    loss = cross_entropy(logits, t, reduction=reduction, inplace_backward=True, consume_logits=True)
    xr = x.double().requires_grad_(True)
    ref = F.cross_entropy(xr, t, reduction=reduction)
    assert abs(float(loss) - float(ref)) < 2e-3 * (1 + abs(float(ref)))
    (loss * upstream).backward()
    (ref * upstream).backward()
    tol = (1e-2 if dtype == torch.bfloat16 else 2e-3) * xr.grad.abs().max().item() + 1e-6
    assert (src.grad.double() - xr.grad).abs().max().item() < tol
    assert torch.equal(logits.detach(), src.grad)        # written in place: no second (N, C) buffer


def test_cross_entropy_consume_flag_is_ignored_where_it_does_not_apply(status_ok):
    x = torch.randn(16, 50, device="cuda", dtype=torch.float32, requires_grad=True)   # fp32, C % 8 != 0
    t = torch.randint(0, 50, (16,), device="cuda")
    keep = x.detach().clone()
    loss = cross_entropy(x, t, label_smoothing=0.1, consume_logits=True)
    loss.backward()
    assert torch.equal(x.detach(), keep)
    xr = keep.double().requires_grad_(True)
    F.cross_entropy(xr, t, label_smoothing=0.1).backward()
    assert (x.grad.double() - xr.grad).abs().max().item() < 1e-5


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float64])
def test_embedding(dtype, status_ok):
    V, D = 1000, 96
    w = torch.randn(V, D, device="cuda", dtype=dtype).requires_grad_(True)
    idx = torch.randint(0, V, (7, 61), device="cuda")
    idx[0, :20] = 5  # a heavily repeated row
    y = embedding(w, idx, padding_idx=7)
    assert torch.equal(y, w.detach()[idx])
    g = torch.randn_like(y)
    y.backward(g)
    wr = w.detach().double().requires_grad_(True)
    F.embedding(idx, wr, padding_idx=7).backward(g.double())
    tol = {torch.bfloat16: 0.15, torch.float32: 1e-5, torch.float64: 1e-12}[dtype]
    assert (w.grad.double() - wr.grad).abs().max().item() < tol
    # deterministic: a second run gives the same bytes
    w2 = w.detach().clone().requires_grad_(True)
    embedding(w2, idx, padding_idx=7).backward(g)
    assert torch.equal(w.grad, w2.grad)


@pytest.mark.parametrize("op", ["sum", "mean", "max", "min", "argmax", "argmin"])
@pytest.mark.parametrize("shape,axis", [((37, 1000), 1), ((5000, 96), 0), ((16384, 768), 0), ((4, 50, 6), 1), ((3, 70000), 1)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float64])
def test_reduce(op, shape, axis, dtype, status_ok):
    x = torch.randn(shape, device="cuda", dtype=dtype)
    y = reduce_axis(x, axis, op)
    xr = x.double()
    if op in ("argmax", "argmin"):
        ref = getattr(torch, op)(xr, dim=axis)
        assert torch.equal(y, ref)
        return
    ref = getattr(torch, op)(xr, dim=axis)
    ref = ref.values if op in ("max", "min") else ref
    tol = {torch.float32: 1e-3, torch.bfloat16: 0.6, torch.float64: 1e-9}[dtype]
    if op in ("max", "min"):
        tol = 1e-9
    assert (y.double() - ref).abs().max().item() <= tol * (1 + 0.01 * ref.abs().max().item())


def test_bias_grad_fp32_accumulate(status_ok):
    x = torch.randn(16384, 768, device="cuda", dtype=torch.bfloat16)
    out = torch.ones(768, device="cuda", dtype=torch.float32)
    reduce_axis(x, 0, "sum", out=out, accumulate=True)
    ref = x.double().sum(0) + 1
    assert (out.double() - ref).abs().max().item() < 1e-2


def test_cast(status_ok):
    x = torch.randn(1001, device="cuda", dtype=torch.float64)
    for dt in (torch.float32, torch.bfloat16, torch.float16):
        assert torch.equal(ew.cast(x, dt), x.to(dt))
    xb = x.to(torch.bfloat16)
    assert torch.equal(ew.cast(xb, torch.float32), xb.float())


def test_dropout_statistics_and_backward(status_ok):
    from gonn_b200.ops.dropout import dropout
    x = torch.ones(1 << 20, device="cuda", dtype=torch.float32, requires_grad=True)
    y = dropout(x, 0.25)
    keep = (y != 0).float().mean().item()
    assert abs(keep - 0.75) < 5e-3
    assert abs(y.max().item() - 1 / 0.75) < 1e-6
    y.backward(torch.ones_like(y))
    assert torch.equal(x.grad, y.detach())  # same mask regenerated in backward


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_dropout_mask_is_the_same_on_the_vector_and_scalar_paths(dtype, status_ok):
    """A length that is a multiple of the vector width takes the 16-byte kernel, one more element takes
    the scalar kernel: element i gets the same draw on both."""
    from gonn_b200 import lib as L
    n = 1 << 16
    x = torch.randn(n + 1, device="cuda").to(dtype)
    yv, ys = torch.empty(n, device="cuda", dtype=dtype), torch.empty(n + 1, device="cuda", dtype=dtype)
    for out, cnt in ((yv, n), (ys, n + 1)):
        L.call("gb_dropout", L.I(L.dtype_code(dtype)), L.ptr(x), L.ptr(out), L.L(cnt), L.F(0.3), L.L(1234), L.L(77),
               L.stream_ptr())
    assert torch.equal(yv, ys[:n])
    assert 0.68 < (yv != 0).float().mean().item() < 0.72


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_fused_rnn_gates_match_oracle(dtype):
    """LSTM / GRU gate kernels, forward and backward, against the torch expression in fp32."""
    from gonn_b200.ops import rnn as R
    torch.manual_seed(0)
    B, H = 37, 48
    tol = dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)
    gates = torch.randn(B, 4 * H, device="cuda").to(dtype).requires_grad_(True)
    c = torch.randn(B, H, device="cuda").to(dtype).requires_grad_(True)
    h1, c1 = R.lstm_gates(gates, c)
    gf, cf = gates.detach().float().requires_grad_(True), c.detach().float().requires_grad_(True)
    h2, c2 = R.lstm_gates_ref(gf, cf)
    dh, dc = torch.randn_like(h2), torch.randn_like(c2)
    g1 = torch.autograd.grad((h1, c1), (gates, c), (dh.to(dtype), dc.to(dtype)))
    g2 = torch.autograd.grad((h2, c2), (gf, cf), (dh, dc))
    assert torch.allclose(h1.float(), h2, **tol) and torch.allclose(c1.float(), c2, **tol)
    for a, b in zip(g1, g2):
        assert torch.allclose(a.float(), b, **tol)
    xg = torch.randn(B, 3 * H, device="cuda").to(dtype).requires_grad_(True)
    hg = torch.randn(B, 3 * H, device="cuda").to(dtype).requires_grad_(True)
    h = torch.randn(B, H, device="cuda").to(dtype).requires_grad_(True)
    y1 = R.gru_gates(xg, hg, h)
    ref_in = [t.detach().float().requires_grad_(True) for t in (xg, hg, h)]
    y2 = R.gru_gates_ref(*ref_in)
    dy = torch.randn_like(y2)
    g1 = torch.autograd.grad(y1, (xg, hg, h), dy.to(dtype))
    g2 = torch.autograd.grad(y2, ref_in, dy)
    assert torch.allclose(y1.float(), y2, **tol)
    for a, b in zip(g1, g2):
        assert torch.allclose(a.float(), b, **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float64])
def test_transpose_and_cumsum_kernels(dtype):
    from gonn_b200.ops.shape import cumsum, transpose_last2
    torch.manual_seed(0)
    x = torch.randn(3, 45, 70, device="cuda").to(dtype)
    assert torch.equal(transpose_last2(x), x.transpose(1, 2).contiguous())
    for axis, n in ((-1, 70), (1, 45)):
        xr = x.detach().clone().requires_grad_(True)
        y = cumsum(xr, axis)
        ref = torch.cumsum(x.double(), dim=axis)
        tol = 1e-10 if dtype == torch.float64 else (1e-4 if dtype == torch.float32 else 0.15)
        assert (y.double() - ref).abs().max().item() <= tol * max(1.0, ref.abs().max().item())
        g = torch.randn_like(x)
        (gx,) = torch.autograd.grad(y, xr, g)
        gref = torch.flip(torch.cumsum(torch.flip(g.double(), [axis]), dim=axis), [axis])
        assert (gx.double() - gref).abs().max().item() <= tol * max(1.0, gref.abs().max().item())
    # a row longer than one chunk (carry across chunks)
    long = torch.randn(2, 5000, device="cuda", dtype=torch.float32)
    assert torch.allclose(cumsum(long, -1), torch.cumsum(long, -1), rtol=1e-4, atol=1e-3)

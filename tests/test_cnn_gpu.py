"""Convolution (im2col by index map + tcgen05 GEMM), pooling and BatchNorm kernels against
torch fp32 / fp64 references; the CNN end to end."""
import pytest
import torch

from gonn_b200.nn.batchnorm import BatchNorm2d
from gonn_b200.nn.conv import Conv1d, Conv2d, Conv3d, ConvTranspose2d
from gonn_b200.nn.pool import AdaptiveAvgPool2d, AvgPool2d, LPPool2d, MaxPool2d

pytestmark = pytest.mark.gpu
F = torch.nn.functional


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("kw", [dict(), dict(stride=2, padding=1), dict(dilation=2, padding=2), dict(groups=2),
                                dict(padding=1, padding_mode="reflect")])
def test_conv2d(dtype, kw, status_ok):
    torch.manual_seed(0)
    c = Conv2d(4, 8, 3, dtype=dtype, device="cuda", **kw)
    x = torch.randn(3, 4, 11, 9, device="cuda", dtype=dtype, requires_grad=True)
    y = c(x)
    xr = x.detach().double().requires_grad_(True)
    w, b = c.weight.detach().double().requires_grad_(True), c.bias.detach().double().requires_grad_(True)
    pm = kw.get("padding_mode", "zeros")
    if pm == "zeros":
        ref = F.conv2d(xr, w, b, stride=kw.get("stride", 1), padding=kw.get("padding", 0),
                       dilation=kw.get("dilation", 1), groups=kw.get("groups", 1))
    else:
        p = kw["padding"]
        ref = F.conv2d(F.pad(xr, (p, p, p, p), mode=pm), w, b)
    tol = 5e-2 if dtype == torch.bfloat16 else 1e-4
    assert (y.double() - ref).abs().max().item() < tol
    g = torch.randn_like(y)
    y.backward(g)
    ref.backward(g.double())
    assert (x.grad.double() - xr.grad).abs().max().item() < tol * 4
    assert (c.weight.grad.double() - w.grad).abs().max().item() < tol * 20
    assert (c.bias.grad.double() - b.grad).abs().max().item() < tol * 30


@pytest.mark.parametrize("case", [
    dict(nd=2, cin=3, cout=64, k=3, hw=(32, 32), n=8),                       # K = 27: one padded k-block
    dict(nd=2, cin=64, cout=128, k=3, hw=(15, 15), n=6),                     # K = 576: nine k-blocks
    dict(nd=2, cin=20, cout=192, k=3, hw=(19, 23), n=3, stride=2, padding=1),  # two M tiles, ragged everything
    dict(nd=2, cin=8, cout=16, k=5, hw=(40, 40), n=2, padding=2, dilation=2),
    dict(nd=1, cin=16, cout=24, k=7, hw=(300,), n=4, padding=3),
    dict(nd=3, cin=4, cout=8, k=3, hw=(6, 7, 8), n=2, padding=1),
    # contractions of at most 32 with a channel count that is a multiple of 4: the direct forward kernel
    dict(nd=2, cin=1, cout=8, k=5, hw=(28, 28), n=5, padding=2, stride=2),   # K = 25, padded borders
    dict(nd=1, cin=2, cout=12, k=9, hw=(301,), n=3, padding=4),              # K = 18, ragged last block of positions
    dict(nd=2, cin=3, cout=64, k=3, hw=(7, 300), n=2),                       # more than 256 positions per row of CTAs
    # ... and 32 / 64 / 128 output channels: the direct weight-gradient kernel as well
    dict(nd=2, cin=3, cout=32, k=3, hw=(20, 20), n=3, padding=1),
    dict(nd=2, cin=2, cout=128, k=3, hw=(9, 11), n=5),
    dict(nd=2, cin=3, cout=64, k=3, hw=(32, 32), n=40),                      # more positions than one pass of the CTAs
])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_implicit_gemm_conv(case, dtype, status_ok):
    """The implicit-GEMM kernels (forward, data gradient, weight gradient over the whole batch)
    against torch's float32 convolution of the same 16-bit values: each output within a 16-bit
    rounding step of its own size plus the fp32 accumulation error."""
    torch.manual_seed(1)
    nd = case["nd"]
    Conv = {1: Conv1d, 2: Conv2d, 3: Conv3d}[nd]
    fconv = {1: F.conv1d, 2: F.conv2d, 3: F.conv3d}[nd]
    kw = {k: case[k] for k in ("stride", "padding", "dilation") if k in case}
    c = Conv(case["cin"], case["cout"], case["k"], dtype=dtype, device="cuda", **kw)
    x = torch.randn(case["n"], case["cin"], *case["hw"], device="cuda", dtype=dtype, requires_grad=True)
    y = c(x)
    xr = x.detach().float().requires_grad_(True)
    w, b = c.weight.detach().float().requires_grad_(True), c.bias.detach().float().requires_grad_(True)
    ref = fconv(xr, w, b, **kw)
    step = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11

    def close(a, r, extra):
        assert a.shape == r.shape
        bad = (a.float() - r).abs() - (2 * step * r.abs() + extra)
        assert bad.max().item() <= 0, bad.max().item()

    close(y, ref, 1e-3)
    g = torch.randn_like(y)
    y.backward(g)
    ref.backward(g.float())
    close(x.grad, xr.grad, 2e-3)
    # the weight gradient sums n * L products: allow the fp32 accumulation error of that many terms
    close(c.weight.grad, w.grad, 2e-3 * (w.grad.abs().max().item() + 1))
    close(c.bias.grad, b.grad, 2e-3 * (b.grad.abs().max().item() + 1))
    # identical bytes from run to run (fixed split order in the weight gradient)
    c.weight.grad = None
    x2 = x.detach().clone().requires_grad_(True)
    c(x2).backward(g)
    assert torch.equal(x2.grad, x.grad)


def test_conv1d_3d_transpose(status_ok):
    torch.manual_seed(0)
    c1 = Conv1d(3, 5, 4, stride=2, device="cuda")
    x1 = torch.randn(2, 3, 17, device="cuda")
    assert (c1(x1) - F.conv1d(x1, c1.weight, c1.bias, stride=2)).abs().max().item() < 1e-4
    c3 = Conv3d(2, 4, 2, device="cuda")
    x3 = torch.randn(2, 2, 5, 6, 7, device="cuda")
    assert (c3(x3) - F.conv3d(x3, c3.weight, c3.bias)).abs().max().item() < 1e-4
    ct = ConvTranspose2d(4, 6, 3, stride=2, padding=1, output_padding=1, device="cuda")
    x = torch.randn(2, 4, 7, 5, device="cuda")
    assert (ct(x) - F.conv_transpose2d(x, ct.weight, ct.bias, stride=2, padding=1, output_padding=1)).abs().max().item() < 1e-4


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_pools(dtype, status_ok):
    x = torch.randn(3, 5, 13, 10, device="cuda", dtype=dtype, requires_grad=True)
    xr = x.detach().float().requires_grad_(True)
    cases = [(MaxPool2d(3, 2, 1), lambda t: F.max_pool2d(t, 3, 2, 1)),
             (MaxPool2d(2), lambda t: F.max_pool2d(t, 2)),
             (AvgPool2d(2, ceil_mode=True, count_include_pad=False), lambda t: F.avg_pool2d(t, 2, ceil_mode=True, count_include_pad=False)),
             (AvgPool2d(3, 1, 1), lambda t: F.avg_pool2d(t, 3, 1, 1)),
             (AdaptiveAvgPool2d(1), lambda t: F.adaptive_avg_pool2d(t, 1)),
             (AdaptiveAvgPool2d((4, 3)), lambda t: F.adaptive_avg_pool2d(t, (4, 3)))]
    for mod, ref_fn in cases:
        x.grad = None
        xr.grad = None
        y = mod(x)
        ref = ref_fn(xr)
        tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
        assert (y.float() - ref).abs().max().item() < tol
        g = torch.randn_like(ref)
        y.backward(g.to(dtype))
        ref.backward(g)
        assert (x.grad.float() - xr.grad).abs().max().item() < tol * 4


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_batchnorm_train_eval(dtype, status_ok):
    x = (torch.randn(8, 6, 7, 5, device="cuda") * 2 + 1).to(dtype).requires_grad_(True)
    bn = BatchNorm2d(6, dtype=dtype, device="cuda")
    with torch.no_grad():
        bn.weight.copy_(torch.rand(6) + 0.5)
        bn.bias.copy_(torch.randn(6))
    tb = torch.nn.BatchNorm2d(6).cuda().double()
    tb.weight.data.copy_(bn.weight.data.double())
    tb.bias.data.copy_(bn.bias.data.double())
    xr = x.detach().double().requires_grad_(True)
    y, yr = bn(x), tb(xr)
    tol = 4e-2 if dtype == torch.bfloat16 else 1e-4
    assert (y.double() - yr).abs().max().item() < tol
    assert (bn.running_mean.double() - tb.running_mean).abs().max().item() < 1e-3
    assert (bn.running_var.double() - tb.running_var).abs().max().item() < 2e-3
    g = torch.randn_like(yr)
    y.backward(g.to(dtype))
    yr.backward(g)
    assert (x.grad.double() - xr.grad).abs().max().item() < tol * 2
    assert (bn.weight.grad.double() - tb.weight.grad).abs().max().item() < tol * 40
    assert (bn.bias.grad.double() - tb.bias.grad).abs().max().item() < tol * 40
    bn.eval(); tb.eval()
    assert (bn(x).double() - tb(xr)).abs().max().item() < tol


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(8, 6, 7, 5), (16, 64, 30, 30), (4, 3, 9, 9)])
def test_batchnorm_with_fused_relu(dtype, shape, status_ok):
    """BatchNorm with the ReLU inside its kernels: the backward masks the incoming gradient where the
    output is zero inside the reduction and apply kernels (no separate elementwise launches)."""
    C = shape[1]
    x = (torch.randn(*shape, device="cuda") * 2 + 0.3).to(dtype).requires_grad_(True)
    bn = BatchNorm2d(C, fused_relu=True, dtype=dtype, device="cuda")
    with torch.no_grad():
        bn.weight.copy_(torch.rand(C) + 0.5)
        bn.bias.copy_(torch.randn(C) * 0.5)
    tb = torch.nn.BatchNorm2d(C).cuda().double()
    tb.weight.data.copy_(bn.weight.data.double())
    tb.bias.data.copy_(bn.bias.data.double())
    xr = x.detach().double().requires_grad_(True)
    y, yr = bn(x), torch.relu(tb(xr))
    tol = 4e-2 if dtype == torch.bfloat16 else 1e-4
    assert (y.double() - yr).abs().max().item() < tol
    g = torch.randn_like(yr)
    # an element that rounds to zero in 16 bits is inactive for the kernel but active for the fp64 reference:
    # no upstream gradient where the two disagree, so that the comparison is about the masking itself
    g = g * ((y.detach() > 0) == (yr.detach() > 0)).double()
    y.backward(g.to(dtype))
    yr.backward(g)
    n = x.numel() / C
    assert (x.grad.double() - xr.grad).abs().max().item() < tol * 2
    assert (bn.weight.grad.double() - tb.weight.grad).abs().max().item() < tol * 4 * n ** 0.5
    assert (bn.bias.grad.double() - tb.bias.grad).abs().max().item() < tol * 4 * n ** 0.5


def test_cnn_trains(status_ok):
    from gonn_b200.distributed.ddp import DistributedDataParallel
    from gonn_b200.models.cnn import SmallCNN
    torch.manual_seed(0)
    m = SmallCNN(dtype=torch.bfloat16, device="cuda")
    ddp = DistributedDataParallel(m, optimizer=dict(kind="adamw", lr=2e-3, weight_decay=0.0))
    x = torch.randn(64, 3, 32, 32, device="cuda", dtype=torch.bfloat16)
    y = torch.randint(0, 10, (64,), device="cuda")
    losses = []
    for _ in range(12):
        loss = m.loss(x, y)
        loss.backward()
        ddp.step()
        losses.append(loss.item())
    assert losses[-1] < losses[0] - 0.3, losses

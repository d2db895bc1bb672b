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

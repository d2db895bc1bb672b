"""int8 tcgen05 GEMM with the dequantising epilogue, device-side observers and fake quantisation
against the host restatement of the reference's integer loop."""
import pytest
import torch

from gonn_b200 import quant as Q
from gonn_b200.nn import Linear

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("per_channel", [False, True])
@pytest.mark.parametrize("shape", [(64, 128, 96), (300, 200, 130), (1024, 768, 3072)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dynamic_linear_matches_integer_reference(per_channel, shape, dtype, status_ok):
    M, K, N = shape
    torch.manual_seed(0)
    lin = Linear(K, N, dtype=torch.float32)
    x = torch.randn(M, K) * 2
    dl = Q.DynamicLinear(lin, per_channel)
    xd = x.to("cuda", dtype)
    y = dl(xd)
    # host reference with the q-parameters of the (dtype-rounded) input
    xr = xd.double().cpu()
    sx, zx = Q.affine_qparams(float(xr.min()), float(xr.max()))
    ref = dl.core.forward_host(xr, sx, zx)
    tol = 2e-2 if dtype == torch.bfloat16 else 2e-4
    assert ((y.double().cpu() - ref).abs() / (1 + ref.abs())).max().item() < tol
    f = lin(x.double().float())
    assert (y.float().cpu() - f).abs().max().item() < 0.06 * f.abs().max().item()


def test_static_linear_and_observer(status_ok):
    torch.manual_seed(1)
    lin = Linear(256, 64)
    sl = Q.StaticLinear(lin, True)
    x = torch.randn(128, 256)
    sl.Calibrate(x)
    y = sl(x.cuda())
    ref = sl.core.forward_host(x.double(), sl.InScale, sl.InZeroPoint)
    assert (y.double().cpu() - ref).abs().max().item() < 1e-3
    qp4, zp = Q._observe_device(x.cuda())
    s, z = Q.affine_qparams(float(x.min()), float(x.max()))
    assert abs(qp4[2].item() - s) < 1e-7 and int(zp.item()) == z


def test_fake_quant_kernel_matches_host(status_ok):
    fq = Q.FakeQuant()
    x = torch.randn(10000) * 2
    fq.train()
    yh = fq(x.double().requires_grad_(True))
    fq.eval()
    xd = x.cuda().requires_grad_(True)
    yd = fq(xd)
    xh = x.double().requires_grad_(True)
    yh = fq(xh)
    assert (yd.double().cpu() - yh).abs().max().item() < 1e-5
    g = torch.randn(10000)
    yd.backward(g.cuda())
    yh.backward(g.double())
    assert (xd.grad.double().cpu() - xh.grad).abs().max().item() < 1e-6

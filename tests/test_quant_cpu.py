"""Quantisation semantics on the host path (quant/*_test.go of the reference): round-trip error
<= scale/2, dynamic int8 Linear close to the float layer, per-channel beats per-tensor, STE
mask, QAT evaluation equals the converted StaticLinear."""
import torch

from gonn_b200 import quant as Q
from gonn_b200.nn import Linear


def test_round_trip_error_within_half_scale():
    t = torch.randn(1000, dtype=torch.float64) * 3
    q = Q.Quantize(t)
    assert (Q.Dequantize(q) - t).abs().max().item() <= q.Scale / 2 + 1e-12
    assert q.Data.dtype == torch.int8 and -128 <= int(q.Data.min()) and int(q.Data.max()) <= 127


def test_round_is_half_away_from_zero_and_affine_includes_zero():
    assert Q.quantize_value(torch.tensor([0.5, -0.5, 1.5, -2.5]), 1.0, 0).tolist() == [1.0, -1.0, 2.0, -3.0]
    s, zp = Q.affine_qparams(2.0, 6.0)         # range nudged to [0, 6]
    assert abs(s - 6.0 / 255) < 1e-15 and zp == -128
    assert Q.affine_qparams(0.0, 0.0) == (1.0, 0)


def test_per_channel_beats_per_tensor():
    torch.manual_seed(0)
    w = torch.randn(8, 32, dtype=torch.float64) * torch.logspace(-2, 1, 8, dtype=torch.float64)[:, None]
    e_pc = (Q.DequantizePerChannel(Q.QuantizePerChannel(w, 0)) - w).abs().mean().item()
    s = Q.symmetric_qparams(w)
    e_pt = ((Q.quantize_value(w, s, 0) * s) - w).abs().mean().item()
    assert e_pc < e_pt


def test_dynamic_linear_close_to_float():
    torch.manual_seed(1)
    lin = Linear(64, 32, dtype=torch.float64)
    x = torch.randn(16, 64, dtype=torch.float64)
    ref = lin(x)
    for pc in (False, True):
        y = Q.DynamicLinear(lin, pc)(x)
        assert (y - ref).abs().max().item() < 0.05 * ref.abs().max().item()


def test_fake_quant_ste_mask():
    fq = Q.FakeQuant(symmetric=True)
    x = torch.tensor([-3.0, -0.2, 0.1, 0.9, 5.0], dtype=torch.float64, requires_grad=True)
    fq.train()
    y = fq(x)
    fq.eval()
    x2 = torch.tensor([-9.0, 0.3, 9.0], dtype=torch.float64, requires_grad=True)
    fq(x2).sum().backward()
    assert x2.grad.tolist() == [0.0, 1.0, 0.0]     # outside the representable range: no gradient
    assert (y - x).abs().max().item() <= fq.Scale / 2 + 1e-12


def test_qat_eval_equals_converted_static_linear():
    torch.manual_seed(2)
    qat = Q.QATLinear(Linear(16, 8, dtype=torch.float64))
    opt_x = torch.randn(64, 16, dtype=torch.float64)
    qat.train()
    for _ in range(5):
        qat(opt_x)
    qat.eval()
    x = torch.randn(10, 16, dtype=torch.float64)
    conv = qat.Convert()
    assert (qat(x) - conv(x)).abs().max().item() < 1e-10
    names = [n for n, _ in qat.named_parameters()]
    assert names == ["linear.weight", "linear.bias"]
    assert [n for n, _ in qat.named_children()] == ["linear", "weight_fq", "input_fq"]

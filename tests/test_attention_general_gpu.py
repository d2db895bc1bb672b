"""The general fused attention kernels (masks, key padding, dropout, fp32 / fp64, odd head sizes)
against materialised-score math in float32 / float64, forward and backward."""
import math

import pytest
import torch

from gonn_b200 import lib as gl
from gonn_b200.ops.attention import general_attention, masked_attention_ref

pytestmark = pytest.mark.gpu

TOL = {torch.float64: 1e-11, torch.float32: 2e-5, torch.float16: 4e-3, torch.bfloat16: 3e-2}


def _keep(B, H, Tq, Tk, p, seed):
    out = torch.empty(B, H, Tq, Tk, dtype=torch.uint8, device="cuda")
    gl.call("gb_attn_keep_mask", gl.ptr(out), gl.I(B), gl.I(H), gl.I(Tq), gl.I(Tk), gl.D(p), gl.L(seed), gl.stream_ptr())
    return out.bool()


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("case", [
    dict(B=2, Tq=70, Tk=70, H=3, D=64, causal=True),
    dict(B=1, Tq=33, Tk=129, H=2, D=20, mask="float"),
    dict(B=2, Tq=64, Tk=50, H=2, D=128, mask="bool", kpm=True),
    dict(B=2, Tq=45, Tk=45, H=1, D=7, causal=True, kpm=True),
    dict(B=1, Tq=96, Tk=96, H=2, D=32, causal=True, drop=0.25),
    dict(B=2, Tq=40, Tk=72, H=2, D=48, mask="float", kpm=True, drop=0.1),
])
def test_general_attention(case, dtype, status_ok):
    B, Tq, Tk, H, D = (case[k] for k in ("B", "Tq", "Tk", "H", "D"))
    g = torch.Generator(device="cuda").manual_seed(Tq * 7 + D)
    q = torch.randn(B, Tq, H, D, device="cuda", generator=g).to(dtype).requires_grad_(True)
    k = torch.randn(B, Tk, H, D, device="cuda", generator=g).to(dtype).requires_grad_(True)
    v = torch.randn(B, Tk, H, D, device="cuda", generator=g).to(dtype).requires_grad_(True)
    mask = add = None
    if case.get("mask") == "float":
        mask = add = torch.randn(Tq, Tk, device="cuda", generator=g)
    elif case.get("mask") == "bool":
        mask = torch.rand(Tq, Tk, device="cuda", generator=g) < 0.3
        mask[:, 0] = False
        add = mask.float() * -1e30
    kpm = None
    if case.get("kpm"):
        kpm = torch.zeros(B, Tk, dtype=torch.bool, device="cuda")
        kpm[:, Tk - 5:] = True
        kpm[0, 1] = True
    p, seed = case.get("drop", 0.0), 1234
    out = general_attention(q, k, v, case.get("causal", False), None, mask, kpm, p, seed)
    ct = torch.float64 if dtype == torch.float64 else torch.float32
    qr, kr, vr = (t.detach().to(ct).requires_grad_(True) for t in (q, k, v))
    keep = _keep(B, H, Tq, Tk, p, seed) if p > 0 else None
    if keep is not None:
        assert abs(keep.float().mean().item() - (1 - p)) < 0.02
    ref = masked_attention_ref(qr, kr, vr, case.get("causal", False), None, add, kpm, keep, p)
    tol = TOL[dtype]
    assert out.dtype == dtype
    assert (out.to(ct) - ref).abs().max().item() < tol * (1 + ref.abs().max().item())
    do = torch.randn(B, Tq, H, D, device="cuda", generator=g).to(dtype)
    out.backward(do)
    ref.backward(do.to(ct))
    for got, want in ((q.grad, qr.grad), (k.grad, kr.grad), (v.grad, vr.grad)):
        assert (got.to(ct) - want).abs().max().item() < 4 * tol * (1 + want.abs().max().item())
    # run to run: identical bytes (fixed summation order, regenerated dropout mask)
    q2, k2, v2 = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    out2 = general_attention(q2, k2, v2, case.get("causal", False), None, mask, kpm, p, seed)
    out2.backward(do)
    assert torch.equal(out2, out) and torch.equal(q2.grad, q.grad) and torch.equal(k2.grad, k.grad)


def test_forward_masked_module_uses_fused_kernels(status_ok):
    """MultiHeadAttention.ForwardMasked on CUDA (fused) against the same module's tensor-op path on
    the CPU in float64; the native call counter shows the general kernel ran."""
    from gonn_b200.nn.attention import MultiHeadAttention
    torch.manual_seed(0)
    mha_cpu = MultiHeadAttention(48, 4, dtype=torch.float64)
    mha_gpu = MultiHeadAttention(48, 4, dtype=torch.float64, device="cuda")
    mha_gpu.load_state_dict(mha_cpu.state_dict())
    x = torch.randn(2, 19, 48, dtype=torch.float64)
    y = torch.randn(2, 23, 48, dtype=torch.float64)
    mask = torch.rand(19, 23) < 0.2
    kpm = torch.zeros(2, 23, dtype=torch.bool)
    kpm[1, 20:] = True
    want = mha_cpu.ForwardMasked(x, y, y, attn_mask=mask, key_padding_mask=kpm)
    n0 = gl.launch_count
    got = mha_gpu.ForwardMasked(x.cuda(), y.cuda(), y.cuda(), attn_mask=mask.cuda(), key_padding_mask=kpm.cuda())
    assert gl.launch_count > n0
    assert (got.cpu() - want).abs().max().item() < 1e-10
    mha_gpu.eval()
    again = mha_gpu.ForwardMasked(x.cuda(), y.cuda(), y.cuda(), attn_mask=mask.cuda(), key_padding_mask=kpm.cuda(),
                                  attn_dropout=0.5)
    assert torch.equal(again, got)          # dropout is inactive in evaluation mode


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32, torch.bfloat16])
def test_misaligned_strided_views_match_contiguous(dtype, status_ok):
    """Views that start one element into a wider buffer cannot use 16-byte loads: the kernels then
    stage their tiles element by element and must give the bytes of the aligned path."""
    B, T, H, D = 2, 77, 3, 40
    g = torch.Generator(device="cuda").manual_seed(5)
    wide = [torch.randn(B, T, H, D + 3, device="cuda", generator=g).to(dtype) for _ in range(3)]
    views = [w[..., 1:D + 1].detach().requires_grad_(True) for w in wide]
    dense = [w[..., 1:D + 1].detach().contiguous().requires_grad_(True) for w in wide]
    assert all(v.data_ptr() % 8 != 0 or v.stride(1) % 4 != 0 for v in views)
    do = torch.randn(B, T, H, D, device="cuda", generator=g).to(dtype)
    a = general_attention(*views, True, None, None, None, 0.2, 99)
    b = general_attention(*dense, True, None, None, None, 0.2, 99)
    assert torch.equal(a, b)
    a.backward(do)
    b.backward(do)
    for x, y in zip(views, dense):
        assert torch.equal(x.grad, y.grad)

"""Flash attention kernels against materialised fp32 attention (forward, LSE, backward).
Pattern: benchmark/flashattn/main.go:102-123 (kernel vs CPU reference) and
benchmark/flashbwd/main.go:40-95 (gradient check) of the reference."""
import math

import pytest
import torch

from gonn_b200.ops import attention as A
from gonn_b200.ops.attention import attention_ref, flash_attention, flash_bwd, flash_fwd

pytestmark = pytest.mark.gpu

CASES = [(1, 128, 1, 128, False), (1, 128, 1, 64, True), (2, 256, 2, 128, True), (2, 512, 3, 64, True),
         (1, 200, 2, 128, True), (1, 333, 1, 64, False), (2, 1024, 4, 128, True),
         # the benchmark shapes' sequence lengths
         (1, 2048, 2, 128, True), (1, 4096, 2, 128, True), (1, 2048, 2, 64, False),
         # head sizes between the two compiled ones: zero-filled by the loads, clipped by the stores
         (2, 256, 2, 32, True), (1, 333, 3, 96, False), (1, 200, 2, 8, True), (2, 128, 1, 40, False),
         (1, 384, 2, 72, True), (1, 256, 2, 112, True)]


@pytest.mark.parametrize("B,S,H,D,causal", CASES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_forward_backward(B, S, H, D, causal, dtype, status_ok):
    q, k, v = (torch.randn(B, S, H, D, device="cuda", dtype=dtype) for _ in range(3))
    scale = 1 / math.sqrt(D)
    out, lse = flash_fwd(q, k, v, causal, scale)
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    ref = attention_ref(qf, kf, vf, causal, scale)
    assert (out.float() - ref).abs().max().item() < 0.02
    s = torch.einsum("bqhd,bkhd->bhqk", qf, kf) * scale
    if causal:
        s = s + torch.triu(torch.ones(S, S, device="cuda"), 1) * -1e30
    assert (lse - torch.logsumexp(s, -1)).abs().max().item() < 1e-3
    do = torch.randn_like(out)
    dq, dk, dv, _ = flash_bwd(q, k, v, out, do, lse, causal, scale)
    ref.backward(do.float())
    for got, want in ((dq, qf.grad), (dk, kf.grad), (dv, vf.grad)):
        assert (got.float() - want).abs().max().item() < 0.01 * want.abs().max().item() + 0.03


def test_strided_qkv_views(status_ok):
    B, S, H, D = 2, 256, 4, 64
    qkv = torch.randn(B, S, 3, H, D, device="cuda", dtype=torch.bfloat16)
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    out = flash_attention(q, k, v, causal=True)
    ref = attention_ref(q.float(), k.float(), v.float(), True)
    assert (out.float() - ref).abs().max().item() < 0.02


def test_cross_attention_lengths(status_ok):
    q = torch.randn(2, 130, 2, 64, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(2, 300, 2, 64, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(2, 300, 2, 64, device="cuda", dtype=torch.bfloat16)
    q.requires_grad_(True)
    out = flash_attention(q, k, v)
    ref = attention_ref(q.float(), k.float(), v.float(), False)
    assert (out.float() - ref).abs().max().item() < 0.02
    out.sum().backward()
    assert torch.isfinite(q.grad).all()


def test_deterministic(status_ok):
    q, k, v = (torch.randn(2, 512, 4, 128, device="cuda", dtype=torch.bfloat16) for _ in range(3))
    o1, l1 = flash_fwd(q, k, v, True, 0.1)
    do = torch.randn_like(o1)
    g1 = flash_bwd(q, k, v, o1, do, l1, True, 0.1)[:3]
    o2, l2 = flash_fwd(q, k, v, True, 0.1)
    g2 = flash_bwd(q, k, v, o2, do, l2, True, 0.1)[:3]
    assert torch.equal(o1, o2)
    for a, b in zip(g1, g2):
        assert torch.equal(a, b)


@pytest.mark.parametrize("B,Sq,Sk,H,D,causal", [(2, 512, 512, 3, 64, True), (1, 200, 200, 2, 128, True),
                                                (2, 130, 300, 2, 64, False), (1, 1024, 1024, 2, 64, True),
                                                (1, 333, 333, 1, 96, False), (2, 192, 192, 2, 64, True)])
def test_backward_with_and_without_the_dS_workspace(B, Sq, Sk, H, D, causal, status_ok):
    """The two ways to get dQ (one product with the spilled dS^T; a second pass that recomputes the
    scores) give the same dK / dV bit for bit and the same dQ up to the summation order, and both
    match fp32 attention."""
    q = torch.randn(B, Sq, H, D, device="cuda", dtype=torch.bfloat16)
    k, v = (torch.randn(B, Sk, H, D, device="cuda", dtype=torch.bfloat16) for _ in range(2))
    scale = 1 / math.sqrt(D)
    out, lse = flash_fwd(q, k, v, causal, scale)
    do = torch.randn_like(out)
    old = A.DS_SPILL_LIMIT_BYTES
    try:
        A.set_ds_spill_limit(1 << 30)
        g_spill = flash_bwd(q, k, v, out, do, lse, causal, scale)[:3]
        A.set_ds_spill_limit(0)
        g_two = flash_bwd(q, k, v, out, do, lse, causal, scale)[:3]
    finally:
        A.set_ds_spill_limit(old)
    assert torch.equal(g_spill[1], g_two[1]) and torch.equal(g_spill[2], g_two[2])
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    attention_ref(qf, kf, vf, causal, scale).backward(do.float())
    for got in (g_spill[0], g_two[0]):
        assert (got.float() - qf.grad).abs().max().item() < 0.01 * qf.grad.abs().max().item() + 0.03
    assert (g_spill[0].float() - g_two[0].float()).abs().max().item() < 0.02 * qf.grad.abs().max().item() + 0.01

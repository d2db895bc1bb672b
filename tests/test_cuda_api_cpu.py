"""Device-buffer API, flat flash-attention entry points and benchmark loops on the host path."""
import math

import numpy as np
import pytest
import torch

from gonn_b200 import cuda as C


def test_device_buffers_and_resident_ops():
    rng = np.random.default_rng(0)
    a, b = rng.standard_normal((5, 7)), rng.standard_normal((7, 3))
    da, db = C.DevUpload(a, device="cpu"), C.DevUpload(b, device="cpu")
    dc = C.DevAlloc(15, device="cpu")
    C.DevMatMul(da, db, dc, 5, 7, 3)
    C.DevSync()
    np.testing.assert_allclose(dc.Download().reshape(5, 3), a @ b, rtol=1e-12)
    v = C.DevUpload([-1.0, 2.0, -3.0], device="cpu")
    w = C.DevAlloc(3, device="cpu")
    C.DevAdd(v, v, w, 3)
    C.DevReLU(w, 3)
    assert w.Download().tolist() == [0.0, 4.0, 0.0]
    w.Free()
    with pytest.raises(RuntimeError):
        w.Download()
    with pytest.raises(ValueError):
        C.DevMatMul(da, db, C.DevAlloc(4, device="cpu"), 5, 7, 3)


def test_f16_buffers_round_and_accumulate_in_fp32():
    rng = np.random.default_rng(1)
    a, b = rng.standard_normal((8, 16)), rng.standard_normal((16, 8))
    da, db = C.DevUploadF16(a, device="cpu"), C.DevUploadF16(b, device="cpu")
    dc = C.DevAllocF16(64, device="cpu")
    assert da.t.dtype == torch.float16
    C.DevMatMulF16(da, db, dc, 8, 16, 8)
    ref = (torch.tensor(a).half().float() @ torch.tensor(b).half().float()).half().double().numpy()
    np.testing.assert_allclose(dc.Download().reshape(8, 8), ref, rtol=0, atol=2e-3)


@pytest.mark.parametrize("causal", [False, True])
def test_flat_flash_attention_matches_autograd(causal):
    BH, S, d = 3, 10, 8
    g = torch.Generator().manual_seed(2)
    Q, K, V, dO = (torch.randn(BH, S, d, dtype=torch.float64, generator=g) for _ in range(4))
    O, L = C.FlashAttnFwd(Q, K, V, BH, S, d, None, causal, device="cpu")
    assert torch.equal(O, C.FlashAttn(Q, K, V, BH, S, d, None, causal, device="cpu"))
    q, k, v = (t.clone().requires_grad_(True) for t in (Q, K, V))
    s = q @ k.transpose(1, 2) / math.sqrt(d)
    if causal:
        s = s + torch.triu(torch.ones(S, S, dtype=torch.float64), 1) * -1e30
    ref = torch.softmax(s, -1) @ v
    torch.testing.assert_close(O, ref, rtol=1e-10, atol=1e-12)
    torch.testing.assert_close(L, torch.logsumexp(s, -1).detach(), rtol=1e-10, atol=1e-12)
    ref.backward(dO)
    dQ, dK, dV = C.FlashAttnBwd(Q, K, V, O, L, dO, BH, S, d, None, causal, device="cpu")
    for got, want in ((dQ, q.grad), (dK, k.grad), (dV, v.grad)):
        torch.testing.assert_close(got, want, rtol=1e-9, atol=1e-11)
    # flat host arrays and device buffers are accepted as well
    O2 = C.FlashAttn(C.DevUpload(Q.numpy(), device="cpu"), K.numpy(), V.reshape(-1).tolist(), BH, S, d,
                     None, causal, device="cpu")
    torch.testing.assert_close(O2, O)


def test_bench_loops_return_positive_times():
    assert C.BenchMatMulDev(16, 16, 16, 2, device="cpu") > 0
    assert C.BenchMatMulDev(16, 16, 16, 2, f32=True, device="cpu") > 0
    assert C.BenchMatMulF16Dev(16, 16, 16, 2, dtype=torch.bfloat16, device="cpu") > 0
    assert C.BenchAddDev(1000, 2, device="cpu") > 0
    assert C.BenchFlashAttn(2, 16, 8, 2, causal=True, device="cpu") > 0


def test_availability_without_a_device():
    if not torch.cuda.is_available():
        assert not C.Available()
        with pytest.raises(RuntimeError):
            C.Backend()
        with pytest.raises(RuntimeError):
            C.DevAlloc(4)


def test_resident_mlp_benchmark_agrees_with_the_tensor_api():
    from gonn_b200.utils.microbench import bench_resident_mlp
    rec = bench_resident_mlp(device="cpu", iters=1)
    assert rec["max_abs_diff"] == 0.0 and rec["resident_ms"] > 0 and rec["eager_ms"] > 0

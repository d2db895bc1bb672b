"""The device-buffer API, the in-library benchmark loops and the tracer's device timing on a GPU
(the host-side behaviour of the same calls is covered by test_cuda_api_cpu.py)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_resident_buffers_match_numpy(status_ok):
    from gonn_b200 import cuda as C
    assert C.Available()
    rng = np.random.default_rng(0)
    m, k, n = 96, 130, 72
    a, b = rng.standard_normal((m, k)), rng.standard_normal((k, n))
    da, db, dc = C.DevUpload(a), C.DevUpload(b), C.DevAlloc(m * n)
    C.DevMatMul(da, db, dc, m, k, n)
    C.DevSync()
    assert np.abs(dc.Download().reshape(m, n) - a @ b).max() < 1e-11
    x, y = rng.standard_normal(5000), rng.standard_normal(5000)
    dx, dy, dz = C.DevUpload(x), C.DevUpload(y), C.DevAlloc(5000)
    C.DevAdd(dx, dy, dz, 5000)
    assert np.abs(dz.Download() - (x + y)).max() == 0
    C.DevReLU(dz, 5000)
    assert np.abs(dz.Download() - np.maximum(x + y, 0)).max() == 0
    # 16-bit storage, fp32 accumulation on the tensor cores
    ha, hb, hc = C.DevUploadF16(a), C.DevUploadF16(b), C.DevAllocF16(m * n)
    C.DevMatMulF16(ha, hb, hc, m, k, n)
    assert np.abs(hc.Download().reshape(m, n) - a @ b).max() < 0.05 * np.abs(a @ b).max()
    for buf in (da, db, dc, dx, dy, dz, ha, hb, hc):
        buf.Free()
    with pytest.raises(RuntimeError):
        da.Download()


def test_in_library_benchmark_loops_return_times(status_ok):
    from gonn_b200 import cuda as C
    assert 0 < C.BenchMatMulF16Dev(512, 512, 512, 3) < 50
    assert 0 < C.BenchMatMulF16Dev(512, 512, 512, 3, dtype=torch.bfloat16) < 50
    assert 0 < C.BenchMatMulDev(512, 512, 512, 3, True) < 50          # fp32: three-plane tensor-core path
    assert 0 < C.BenchMatMulDev(512, 512, 512, 3, False) < 50         # fp64: tensor-core fp64
    assert 0 < C.BenchAddDev(1 << 20, 3, True) < 50
    assert 0 < C.BenchAddDev(1 << 20, 3, False) < 50
    assert 0 < C.BenchFlashAttn(8, 256, 64, 3, True) < 50             # bf16 tcgen05 kernel
    assert 0 < C.BenchFlashAttn(4, 128, 64, 3, False, dtype=torch.float64) < 500   # general fp64 kernel


def test_float64_attention_entry_points_match_float64_math(status_ok):
    from gonn_b200 import cuda as C
    BH, S, d = 6, 50, 24
    g = torch.Generator().manual_seed(0)
    q, k, v, do = (torch.randn(BH, S, d, dtype=torch.float64, generator=g) for _ in range(4))
    o, L = C.FlashAttnFwd(q, k, v, BH, S, d, None, True, dtype=torch.float64)
    dq, dk, dv = C.FlashAttnBwd(q, k, v, o, L, do, BH, S, d, None, True, dtype=torch.float64)
    qr, kr, vr = (t.clone().requires_grad_(True) for t in (q, k, v))
    s = torch.matmul(qr, kr.transpose(1, 2)) / d ** 0.5
    s = s.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool), 1), -1e30)
    ref = torch.matmul(torch.softmax(s, -1), vr)
    ref.backward(do)
    assert (o.cpu() - ref).abs().max().item() < 1e-12
    assert (L.cpu() - torch.logsumexp(s, -1)).abs().max().item() < 1e-12
    for got, want in ((dq, qr.grad), (dk, kr.grad), (dv, vr.grad)):
        assert (got.cpu() - want).abs().max().item() < 1e-11


def test_tracer_device_time_and_nvtx(status_ok):
    from gonn_b200.ops.gemm import gemm
    from gonn_b200.ops.norm import layer_norm
    from gonn_b200.utils.trace import Tracer
    a = torch.randn(1024, 1024, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(1024, device="cuda", dtype=torch.bfloat16)
    with Tracer(device_time=True, nvtx=True) as tr:
        for _ in range(3):
            layer_norm(gemm(a, a), w, None)
    tr.finish()
    rows = {r["name"]: r for r in tr.summary()}
    assert rows["gb_gemm16"]["calls"] == 3 and rows["gb_norm_fwd"]["calls"] == 3
    assert all(r["device_ms"] > 0 for r in rows.values())
    assert "gb_gemm16" in tr.table()
    assert len(tr.chrome_trace()["traceEvents"]) >= 6

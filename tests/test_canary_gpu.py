"""Kernels that write into caller-provided buffers, run on canary-padded outputs at ragged sizes:
a store before the start or past the end of an output changes a guard byte and fails the test.
This is one of the stand-ins for a memory checker (the other is the bounds-checked build)."""
import math

import pytest
import torch

from gonn_b200.utils.canary import guarded

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32, torch.float64])
@pytest.mark.parametrize("M,N,K", [(129, 72, 200), (1000, 264, 136), (64, 8, 64), (257, 513, 72)])
def test_gemm_outputs_stay_inside(dtype, M, N, K):
    from gonn_b200.ops.gemm import gemm
    a = torch.randn(M, K, device="cuda", dtype=dtype)
    b = torch.randn(K, N, device="cuda", dtype=dtype)
    out = guarded((M, N), dtype, fill=0.0)
    gemm(a, b, out=out.t)
    out.check(f"gemm {M}x{N}x{K} {dtype}")
    ref = a.double() @ b.double()
    tol = {torch.bfloat16: 2e-2, torch.float16: 4e-3, torch.float32: 1e-5, torch.float64: 1e-12}[dtype]
    assert ((out.t.double() - ref).abs().max() / ref.abs().max()).item() < tol


@pytest.mark.parametrize("rows,D,dtype", [(37, 768, torch.bfloat16), (1000, 1001, torch.float32),
                                          (4099, 520, torch.bfloat16), (513, 4096, torch.float32)])
def test_norm_outputs_stay_inside(rows, D, dtype):
    from gonn_b200 import lib as L
    lib = L.lib()
    x = torch.randn(rows, D, device="cuda").to(dtype)
    dy = torch.randn(rows, D, device="cuda").to(dtype)
    w = (torch.randn(D, device="cuda") * 0.2 + 1).to(dtype)
    b = torch.zeros(D, device="cuda", dtype=dtype)
    y, dx = guarded((rows, D), dtype), guarded((rows, D), dtype)
    mean, rstd = guarded((rows,), torch.float32), guarded((rows,), torch.float32)
    dg, db = guarded((D,), dtype), guarded((D,), dtype)
    srows = lib.gb_norm_bwd_scratch_rows()
    scratch = guarded((srows * 2 * D,), torch.float32)
    dt, s = L.dtype_code(dtype), L.stream_ptr()
    assert lib.gb_norm_fwd(L.I(0), L.I(dt), L.I(dt), L.ptr(x), L.ptr(w), L.ptr(b), L.ptr(y.t), L.ptr(mean.t),
                           L.ptr(rstd.t), L.L(rows), L.I(D), L.F(1e-5), s) == 0
    assert lib.gb_norm_bwd(L.I(0), L.I(dt), L.I(dt), L.ptr(x), L.ptr(dy), L.ptr(w), L.ptr(mean.t), L.ptr(rstd.t),
                           L.ptr(dx.t), L.ptr(dg.t), L.ptr(db.t), L.ptr(scratch.t), L.I(srows), L.L(rows), L.I(D), s) == 0
    for name, g in (("y", y), ("dx", dx), ("mean", mean), ("rstd", rstd), ("dgamma", dg), ("dbeta", db),
                    ("scratch", scratch)):
        g.check(f"layer norm {rows}x{D} {dtype}: {name}")
    ref = torch.nn.functional.layer_norm(x.float(), (D,), w.float(), b.float(), 1e-5)
    assert (y.t.float() - ref).abs().max().item() < (5e-2 if dtype == torch.bfloat16 else 1e-4)
    L.assert_status_ok()


@pytest.mark.parametrize("n,dtype", [(1, torch.float32), (1023, torch.bfloat16), (65537, torch.float32),
                                     (1000003, torch.bfloat16), (4097, torch.float64)])
def test_elementwise_outputs_stay_inside(n, dtype):
    from gonn_b200.ops import elementwise as ew
    a = torch.randn(n, device="cuda").to(dtype)
    b = torch.randn(n, device="cuda").to(dtype)
    from gonn_b200 import lib as L
    out = guarded((n,), dtype)
    L.call("gb_binary", L.I(0), L.I(L.dtype_code(dtype)), L.ptr(a), L.ptr(b), L.ptr(out.t), L.L(n), L.I(0),
           L.ptr(None), L.ptr(None), L.ptr(None), L.ptr(None))
    out.check(f"add n={n} {dtype}")
    assert torch.equal(out.t, a + b)
    assert ew is not None


@pytest.mark.parametrize("n,D,V,dtype", [(77, 768, 1000, torch.bfloat16), (513, 100, 50, torch.float32),
                                         (4096, 72, 32000, torch.bfloat16)])
def test_embedding_outputs_stay_inside(n, D, V, dtype):
    from gonn_b200 import lib as L
    lib = L.lib()
    lib.gb_embedding_bwd_scratch_ints.restype = __import__("ctypes").c_longlong
    w = torch.randn(V, D, device="cuda").to(dtype)
    idx = torch.randint(0, V, (n,), device="cuda")
    out = guarded((n, D), dtype)
    L.call("gb_gather_rows", L.I(L.dtype_code(dtype)), L.ptr(w), L.ptr(idx), L.ptr(out.t), L.L(n), L.I(D), L.L(V),
           L.stream_ptr())
    out.check("embedding gather")
    assert torch.equal(out.t, w[idx])
    dy = torch.randn(n, D, device="cuda").to(dtype)
    dw = guarded((V, D), dtype)
    ints = lib.gb_embedding_bwd_scratch_ints(L.L(n), L.L(V))
    scratch = guarded((ints,), torch.int32)
    dt = L.dtype_code(dtype)
    L.call("gb_embedding_bwd", L.I(dt), L.I(dt), L.ptr(dy), L.ptr(idx), L.ptr(dw.t), L.L(n), L.I(D), L.L(V), L.L(-1),
           L.I(0), L.ptr(scratch.t), L.stream_ptr())
    dw.check("embedding backward: table gradient")
    scratch.check("embedding backward: scratch")
    ref = torch.zeros(V, D, device="cuda", dtype=torch.float32).index_add_(0, idx, dy.float())
    assert (dw.t.float() - ref).abs().max().item() < (6e-2 if dtype == torch.bfloat16 else 1e-4)
    L.assert_status_ok()


@pytest.mark.parametrize("B,H,W,k", [(6, 9, 11, 2), (130, 30, 30, 2), (3, 7, 7, 3)])
def test_pooling_outputs_stay_inside(B, H, W, k):
    from gonn_b200 import lib as L
    from gonn_b200.ops import window as win
    x = torch.randn(B, H * W, device="cuda", dtype=torch.bfloat16)
    idx_np, _ = win.sliding_index((H, W), k, k, 0, 1)
    maps = win.device_maps(idx_np, H * W, x.device, True)
    nwin, T = idx_np.shape
    y, arg = guarded((B, nwin), torch.bfloat16), guarded((B, nwin), torch.int32)
    L.call("gb_pool_fwd", L.I(0), L.ptr(x), L.ptr(maps["idx"]), L.ptr(y.t), L.ptr(arg.t), L.L(B), L.L(H * W), L.I(nwin),
           L.I(T), L.I(0), L.I(0), L.F(2.0), L.stream_ptr())
    y.check("max pool forward"); arg.check("max pool arg-max")
    ref = torch.nn.functional.max_pool2d(x.view(B, 1, H, W).float(), k).view(B, -1)
    assert torch.equal(y.t.float(), ref)
    # backward through the disjoint-window table
    dy = torch.randn(B, nwin, device="cuda", dtype=torch.bfloat16)
    dx = guarded((B, H * W), torch.bfloat16)
    L.call("gb_pool_bwd_disjoint", L.I(0), L.ptr(dy), L.ptr(arg.t), L.ptr(maps["p2w"]), L.ptr(maps["wcnt"]),
           L.ptr(dx.t), L.L(B), L.L(H * W), L.I(nwin), L.I(T), L.I(0), L.I(0), L.stream_ptr())
    dx.check("max pool backward")
    assert math.isfinite(float(dx.t.float().sum()))
    L.assert_status_ok()

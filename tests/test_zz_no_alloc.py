"""The allocation-free LayerNorm-backward entry point, called through its exported C symbol.

Some users of the library cannot allocate device memory when they call it (they pass raw
pointers from a foreign runtime, or their memory plan is frozen before the first step), so
``gb_norm_bwd_noalloc`` keeps its scratch in an array inside the library.  This test calls
the symbol directly with ctypes and checks dx / dgamma / dbeta against the regular entry
point (which takes caller-provided scratch), twice in a row, because the built-in array is
shared by all calls and keeps the previous call's contents.

The file name sorts last on purpose: a run that stops at the first failure has then already
run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_pair(lib, L, rows, D, dtype, seed, kind=0, want_params=True):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, D, device="cuda", generator=g).to(dtype)
    dy = torch.randn(rows, D, device="cuda", generator=g).to(dtype)
    w = (torch.randn(D, device="cuda", generator=g) * 0.3 + 1).to(dtype)
    b = torch.zeros(D, device="cuda", dtype=dtype)
    y = torch.empty_like(x)
    mean = None if kind else torch.empty(rows, device="cuda", dtype=torch.float32)   # RMSNorm keeps no mean
    rstd = torch.empty(rows, device="cuda", dtype=torch.float32)
    dt = L.dtype_code(dtype)
    s = L.stream_ptr()
    rc = lib.gb_norm_fwd(L.I(kind), L.I(dt), L.I(dt), L.ptr(x), L.ptr(w), L.ptr(None if kind else b), L.ptr(y),
                         L.ptr(mean), L.ptr(rstd), L.L(rows), L.I(D), L.F(1e-5), s)
    assert rc == 0
    # regular entry point: the caller provides the scratch
    srows = lib.gb_norm_bwd_scratch_rows()
    scratch = torch.empty(srows * 2 * D, device="cuda", dtype=torch.float32)
    def outs():
        dx = torch.empty_like(x)
        if not want_params:
            return dx, None, None
        return dx, torch.empty_like(w), (None if kind else torch.empty_like(w))

    dx0, dg0, db0 = outs()
    rc = lib.gb_norm_bwd(L.I(kind), L.I(dt), L.I(dt), L.ptr(x), L.ptr(dy), L.ptr(w), L.ptr(mean), L.ptr(rstd),
                         L.ptr(dx0), L.ptr(dg0), L.ptr(db0), L.ptr(scratch), L.I(srows), L.L(rows), L.I(D), s)
    assert rc == 0
    # allocation-free entry point: outputs pre-allocated here, nothing allocated inside.  The driver's own
    # count of free device memory must not move either (torch's counter only sees torch's allocator).
    dx1, dg1, db1 = outs()
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    free_before = torch.cuda.mem_get_info()[0]
    rc = lib.gb_norm_bwd_noalloc(L.I(kind), L.I(dt), L.I(dt), L.ptr(x), L.ptr(dy), L.ptr(w), L.ptr(mean),
                                 L.ptr(rstd), L.ptr(dx1), L.ptr(dg1), L.ptr(db1), L.L(rows), L.I(D), s)
    assert rc == 0, lib.gb_last_error()
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    assert torch.cuda.mem_get_info()[0] >= free_before
    return [t for t in (dx0, dg0, db0) if t is not None], [t for t in (dx1, dg1, db1) if t is not None]


def test_noalloc_matches_regular_entry_point_twice():
    from gonn_b200 import lib as L
    lib = L.lib()
    lib.gb_last_error.restype = ctypes.c_char_p
    # two calls in a row with different shapes and data: the second must not see the first's partials
    # one warm-up call first: the entry point's first call on a device looks up the array's address
    _call_pair(lib, L, 64, 256, torch.float32, 99)
    cases = [dict(rows=4096, D=768, dtype=torch.bfloat16), dict(rows=1000, D=2048, dtype=torch.float32),
             dict(rows=600, D=4096, dtype=torch.float32),                  # the widest row: the whole array in use
             dict(rows=300, D=1024, dtype=torch.bfloat16, kind=1),         # RMSNorm: no mean, no bias gradient
             dict(rows=257, D=512, dtype=torch.float32, want_params=False),  # dx only
             dict(rows=129, D=1001, dtype=torch.float32)]                  # odd width: the unvectorised kernels
    for seed, c in enumerate(cases):
        ref, got = _call_pair(lib, L, c["rows"], c["D"], c["dtype"], seed, c.get("kind", 0), c.get("want_params", True))
        assert len(ref) == len(got)
        for a, b in zip(ref, got):
            tol = 3e-2 if c["dtype"] == torch.bfloat16 else 1e-4
            assert ((a.double() - b.double()).abs() / (1 + a.double().abs())).max().item() < tol
    L.assert_status_ok()


def test_noalloc_rejects_rows_wider_than_the_builtin_scratch():
    from gonn_b200 import lib as L
    lib = L.lib()
    lib.gb_last_error.restype = ctypes.c_char_p
    D = lib.gb_norm_bwd_noalloc_max_dim() + 8
    x = torch.zeros(2, D, device="cuda", dtype=torch.float32)
    v = torch.zeros(2, device="cuda", dtype=torch.float32)
    w = torch.ones(D, device="cuda", dtype=torch.float32)
    rc = lib.gb_norm_bwd_noalloc(L.I(0), L.I(2), L.I(2), L.ptr(x), L.ptr(x), L.ptr(w), L.ptr(v), L.ptr(v),
                                 L.ptr(x), L.ptr(w), L.ptr(w), L.L(2), L.I(D), L.stream_ptr())
    assert rc == -5
    assert b"exceeds the built-in scratch" in lib.gb_last_error()

"""In-kernel collectives.  On one GPU the W ranks are emulated inside ONE cooperative
launch (gridDim.y = W), never as separate launches that wait on each other.  The
time-out test makes a wait run out (a flag that nothing sets) and checks the status word;
nothing here faults or hangs a device."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _symm(world, nbytes):
    from gonn_b200.distributed.nvlink import SymmetricMemory
    return SymmetricMemory(nbytes, emulate=world)


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_allreduce_mean_emulated(world, dtype, status_ok):
    n = world * 8 * 1000
    sm = _symm(world, 2 * n + 4096)
    grads = [torch.randn(n, device="cuda").to(dtype) for _ in range(world)]
    for r in range(world):
        sm.view(0, n, dtype, rank=r).copy_(grads[r])
    sm.fused_step(0, dtype, 0, 0, n, None, None, None, [0, 0, 0, 0, 0, 1, 1, 1.0], ctas=8)
    torch.cuda.synchronize()
    # fixed rank-order fp32 sum, then 1/W, then one rounding: exactly what the kernel does
    acc = torch.zeros(n, device="cuda")
    for g in grads:
        acc += g.float()
    want = (acc * (1.0 / world)).to(dtype)
    outs = [sm.view(0, n, dtype, rank=r) for r in range(world)]
    assert torch.equal(outs[0], want)
    for o in outs[1:]:
        assert torch.equal(o, outs[0])  # identical bytes on every rank
    sm.check()


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("dtype,n", [(torch.float32, 260), (torch.bfloat16, 8 * 1000), (torch.float16, 8 * 37),
                                     (torch.float32, 16384)])
def test_oneshot_allreduce_emulated(world, dtype, n, status_ok):
    """Short vectors take the one-shot kernel (push, one barrier, local sum in rank order).  Several
    calls in a row alternate between the two slot sets; every rank must hold identical bytes."""
    sm = _symm(world, 4 * n + 4096)
    for call in range(4):
        vals = [(torch.randn(n, device="cuda") * (call + 1)).to(dtype) for _ in range(world)]
        for r in range(world):
            sm.view(0, n, dtype, rank=r).copy_(vals[r])
        sm.all_reduce(0, n, dtype, "mean" if call % 2 else "sum", ctas=8)
        torch.cuda.synchronize()
        acc = torch.zeros(n, device="cuda")
        for v in vals:
            acc += v.float()
        want = (acc * ((1.0 / world) if call % 2 else 1.0)).to(dtype)
        outs = [sm.view(0, n, dtype, rank=r) for r in range(world)]
        assert torch.allclose(outs[0].float(), want.float(), rtol=1e-6 if dtype == torch.float32 else 1e-2, atol=1e-6)
        for o in outs[1:]:
            assert torch.equal(o, outs[0])
    sm.check()


@pytest.mark.parametrize("world", [2, 8])
def test_allreduce_fp32_sum_emulated(world, status_ok):
    """fp32 buffers through the same two-shot kernel (``all_reduce`` with op sum)."""
    n = world * 8 * 777
    sm = _symm(world, 4 * n + 4096)
    vals = [torch.randn(n, device="cuda") for _ in range(world)]
    for r in range(world):
        sm.view(0, n, torch.float32, rank=r).copy_(vals[r])
    sm.all_reduce(0, n, torch.float32, "sum", ctas=8)
    torch.cuda.synchronize()
    acc = torch.zeros(n, device="cuda")
    for v in vals:
        acc += v
    # the kernel sums in rank order, multiplies by W/W = 1
    outs = [sm.view(0, n, torch.float32, rank=r) for r in range(world)]
    assert torch.allclose(outs[0], acc, rtol=1e-6, atol=1e-6)
    for o in outs[1:]:
        assert torch.equal(o, outs[0])
    sm.check()


@pytest.mark.parametrize("world", [1, 2, 4])
def test_zero1_adamw_step_emulated(world, status_ok):
    from gonn_b200.distributed.nvlink import SymmetricMemory
    n = max(world, 1) * 8 * 512
    dtype = torch.bfloat16
    sm = SymmetricMemory(4 * n + 4096, emulate=world) if world > 1 else SymmetricMemory(4 * n + 4096)
    W = world
    p0 = torch.randn(n, device="cuda")
    grads = [torch.randn(n, device="cuda").to(dtype) for _ in range(W)]
    L = n // W
    masters = [p0[r * L:(r + 1) * L].clone() for r in range(W)]
    ms = [torch.zeros(L, device="cuda") for _ in range(W)]
    vs = [torch.zeros(L, device="cuda") for _ in range(W)]
    goff, poff = 0, 2 * n + 2048
    for r in range(W):
        sm.view(goff, n, dtype, rank=r).copy_(grads[r])
        sm.view(poff, n, dtype, rank=r).copy_(p0.to(dtype))
    lr, wd, b1, b2, eps = 1e-2, 0.1, 0.9, 0.999, 1e-8
    ref_p, ref_m, ref_v = p0.clone(), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    for t in (1, 2):
        hy = [lr, wd, b1, b2, eps, 1 - b1 ** t, 1 - b2 ** t, 1.0]
        if W > 1:
            sm.fused_step(1, dtype, goff, poff, n, masters, ms, vs, hy, ctas=8)
        else:
            sm.fused_step(1, dtype, goff, poff, n, masters[0], ms[0], vs[0], hy, ctas=8)
        g = sum(x.float() for x in grads) / W
        ref_p.mul_(1 - lr * wd)
        ref_m.mul_(b1).add_(g, alpha=1 - b1)
        ref_v.mul_(b2).addcmul_(g, g, value=1 - b2)
        ref_p.sub_(lr * (ref_m / hy[5]) / ((ref_v / hy[6]).sqrt() + eps))
    torch.cuda.synchronize()
    got = [sm.view(poff, n, dtype, rank=r) for r in range(W)]
    assert (got[0].float() - ref_p).abs().max().item() < 2e-2
    assert (torch.cat(masters) - ref_p).abs().max().item() < 1e-5
    for o in got[1:]:
        assert torch.equal(o, got[0])
    sm.check()


def test_small_allreduce_broadcast_barrier_emulated(status_ok):
    W = 4
    sm = _symm(W, 1 << 21)
    vecs = [torch.full((129,), float(r + 1), device="cuda") + torch.arange(129, device="cuda") for r in range(W)]
    want = sum(v.clone() for v in vecs)
    sm.allreduce_small(vecs, 0)
    torch.cuda.synchronize()
    for v in vecs:
        assert torch.equal(v, want)
    off = 1 << 20
    for r in range(W):
        sm.view(off, 4096, torch.float32, rank=r).fill_(float(r))
    sm.broadcast(2, off, 4096 * 4, ctas=4)
    sm.barrier()
    torch.cuda.synchronize()
    for r in range(W):
        assert bool((sm.view(off, 4096, torch.float32, rank=r) == 2.0).all())
    sm.check()


def test_wait_that_runs_out_sets_status_and_keeps_context():
    from gonn_b200 import lib as L
    lib = L.lib()
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    L.read_status()  # clear
    rc = lib.gb_comm_wait_flag(L.ptr(flag), ctypes.c_uint(7), ctypes.c_longlong(50_000_000), L.stream_ptr())
    assert rc == 0
    code, detail, _, count = L.read_status()
    assert code == 3 and detail == 999 and count == 1  # ST_COMM_TIMEOUT
    # the context is still usable and a later wait on a flag that IS set returns cleanly
    flag.fill_(7)
    lib.gb_comm_wait_flag(L.ptr(flag), ctypes.c_uint(7), ctypes.c_longlong(50_000_000), L.stream_ptr())
    assert L.read_status()[0] == 0
    assert float(torch.ones(4, device="cuda").sum()) == 4.0


def test_ddp_single_rank_matches_adamw_reference(status_ok):
    from gonn_b200.distributed.ddp import DistributedDataParallel
    from gonn_b200.models import TransformerLM
    torch.manual_seed(0)
    kw = dict(vocab=512, d_model=128, n_layers=2, n_heads=2, d_ff=256, max_seq=64, dtype=torch.bfloat16)
    model = TransformerLM(device="cuda", **kw)
    ref = TransformerLM(device="cuda", **kw)
    ref.load_state_dict(model.state_dict())
    masters = [p.detach().float().clone() for p in ref.parameters()]
    ddp = DistributedDataParallel(model, optimizer=dict(kind="adamw", lr=1e-3, weight_decay=0.1))
    opt = torch.optim.AdamW(masters, lr=1e-3, weight_decay=0.1, betas=(0.9, 0.999), eps=1e-8)
    ids = torch.randint(0, 512, (4, 64), device="cuda")
    tgt = torch.roll(ids, -1, 1)
    for _ in range(3):
        loss = model.loss(ids, tgt)
        loss.backward()
        ddp.step()
        rl = ref.loss(ids, tgt)
        for p in ref.parameters():
            p.grad = None
        rl.backward()
        for m, p in zip(masters, ref.parameters()):
            m.grad = p.grad.float()
        opt.step()
        with torch.no_grad():
            for m, p in zip(masters, ref.parameters()):
                p.copy_(m.to(p.dtype))
        assert abs(loss.item() - rl.item()) < 2e-2
    for (n, p), q in zip(model.named_parameters(), ref.parameters()):
        assert (p.float() - q.float()).abs().max().item() < 2e-2, n

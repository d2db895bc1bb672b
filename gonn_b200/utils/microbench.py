"""Micro-benchmarks of the kernels, one JSON line per measurement.

    python -m gonn_b200.utils.microbench gemm
    python -m gonn_b200.utils.microbench elementwise
    python -m gonn_b200.utils.microbench flash
    python -m gonn_b200.utils.microbench norm
    python -m gonn_b200.utils.microbench resident                 # the reference's resident-MLP forward benchmark
    python -m gonn_b200.utils.microbench mha                      # the reference's MultiHeadAttention Forward / ForwardFused benchmark
    python -m gonn_b200.utils.microbench refattn                  # the reference's attention benchmark shapes
    python -m gonn_b200.utils.microbench mlp                      # CPU, config of the reference's quick start
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m gonn_b200.utils.microbench allreduce                   # bus-bandwidth sweep, NVLink kernels vs NCCL

The shapes are the ones the reference's own benchmark programs use (square matmul
N = 256..2048 of benchmark/gonn/main.go, elementwise add / relu at 1e6 and 1e7 elements,
attention at (BH, S, d) = (16, 2048, 64), (32, 1024, 64), (64, 512, 64) of
benchmark/flashattn/main.go) plus the shapes of the transformer configurations.

Timing: CUDA events around every call, 3 warm-up calls, the median of the timed calls;
a 256 MB buffer is rewritten between calls so that no operand is served from L2.  Every
line carries the same measurement of the stock PyTorch op for comparison.
"""
from __future__ import annotations

import json
import math
import os
import statistics
import sys
import time

import torch

_flush_buf = None


def _flush():
    global _flush_buf
    if _flush_buf is None:
        _flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _flush_buf.zero_()


def timeit(fn, iters: int = 10, flush: bool = True) -> float:
    """Median device time of ``fn`` in milliseconds."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush:
            _flush()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    return statistics.median(times)


def _emit(**kw):
    print(json.dumps(kw), flush=True)


def bench_gemm():
    from ..ops.gemm import gemm
    shapes = [(n, n, n, "nt") for n in (256, 512, 1024, 2048, 4096, 8192)]
    shapes += [(16384, 768, 768, "nt"), (16384, 2304, 768, "nt"), (16384, 3072, 768, "nt"),
               (16384, 768, 3072, "nt"), (16384, 32000, 768, "nt"), (16384, 768, 3072, "nn"),
               (768, 3072, 16384, "tn"), (2304, 768, 16384, "tn"), (8192, 8192, 2048, "nt"),
               (8192, 2048, 8192, "nn"), (8192, 50304, 2048, "nt"), (2048, 8192, 8192, "tn")]
    for M, N, K, lay in shapes:
        ta, tb = lay[0] == "t", lay[1] == "t"
        a = torch.randn((K, M) if ta else (M, K), device="cuda", dtype=torch.bfloat16)
        b = torch.randn((N, K) if tb else (K, N), device="cuda", dtype=torch.bfloat16)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        A, B = (a.t() if ta else a), (b.t() if tb else b)
        ours = timeit(lambda: gemm(a, b, trans_a=ta, trans_b=tb, out=out))
        ref = timeit(lambda: torch.matmul(A, B, out=out))
        fl = 2.0 * M * N * K
        _emit(bench="gemm", dtype="bf16", M=M, N=N, K=K, layout=lay, ms=ours, tflops=fl / ours / 1e9,
              torch_ms=ref, torch_tflops=fl / ref / 1e9)


def bench_elementwise():
    from ..ops.elementwise import binary, unary
    for dt in (torch.float32, torch.bfloat16):
        for n in (10 ** 6, 10 ** 7, 10 ** 8):
            x = torch.randn(n, device="cuda", dtype=dt)
            y = torch.randn(n, device="cuda", dtype=dt)
            esz = x.element_size()
            t = timeit(lambda: binary("add", x, y))
            r = timeit(lambda: torch.add(x, y))
            _emit(bench="add", dtype=str(dt), n=n, ms=t, gbs=3 * n * esz / t / 1e6, torch_ms=r,
                  torch_gbs=3 * n * esz / r / 1e6)
            t = timeit(lambda: unary("relu", x))
            r = timeit(lambda: torch.relu(x))
            _emit(bench="relu", dtype=str(dt), n=n, ms=t, gbs=2 * n * esz / t / 1e6, torch_ms=r,
                  torch_gbs=2 * n * esz / r / 1e6)


def bench_flash():
    from ..ops.attention import flash_bwd, flash_fwd
    F = torch.nn.functional
    cases = [(8, 4096, 16, 128, True), (8, 4096, 16, 128, False), (16, 1024, 12, 64, True),
             (4, 2048, 16, 128, True), (1, 2048, 16, 64, False), (1, 1024, 32, 64, False),
             (1, 512, 64, 64, False), (1, 2048, 16, 64, True)]
    for B, S, H, D, causal in cases:
        q, k, v = (torch.randn(B, S, H, D, device="cuda", dtype=torch.bfloat16) for _ in range(3))
        scale = 1 / math.sqrt(D)
        out, lse = flash_fwd(q, k, v, causal, scale)
        do = torch.randn_like(out)
        fl = 4.0 * B * H * S * S * D * (0.5 if causal else 1.0)
        tf = timeit(lambda: flash_fwd(q, k, v, causal, scale))
        tb = timeit(lambda: flash_bwd(q, k, v, out, do, lse, causal, scale))
        qt, kt, vt = (t.permute(0, 2, 1, 3).contiguous().requires_grad_(True) for t in (q, k, v))
        o = F.scaled_dot_product_attention(qt, kt, vt, is_causal=causal)
        g = torch.randn_like(o)
        rf = timeit(lambda: F.scaled_dot_product_attention(qt, kt, vt, is_causal=causal))
        rb = timeit(lambda: torch.autograd.grad(o, (qt, kt, vt), g, retain_graph=True))
        _emit(bench="flash", dtype="bf16", B=B, S=S, H=H, D=D, causal=causal, fwd_ms=tf,
              fwd_tflops=fl / tf / 1e9, bwd_ms=tb, bwd_tflops=2.5 * fl / tb / 1e9, torch_fwd_ms=rf,
              torch_bwd_ms=rb, flop_convention="4*B*H*S*S*D, halved when causal; backward 2.5x")


def bench_reference_attention():
    """The reference's attention benchmark (benchmark/flashattn/main.go:127-149): forward attention
    on resident (BH, S, d) inputs for (16, 2048, 64), (32, 1024, 64), (64, 512, 64), causal and
    not, FLOPs = 4 BH S^2 d (halved when causal), through the flat entry points of
    ``gonn_b200.cuda``; each line also checks forward and backward against float64 math."""
    from .. import cuda as C
    F = torch.nn.functional
    for BH, S, d in ((16, 2048, 64), (32, 1024, 64), (64, 512, 64)):
        for causal in (False, True):
            g = torch.Generator(device="cuda").manual_seed(BH + S)
            q, k, v, do = (torch.randn(BH, S, d, device="cuda", dtype=torch.bfloat16, generator=g) for _ in range(4))
            o, lse = C.FlashAttnFwd(q, k, v, BH, S, d, None, causal)
            dq, dk, dv = C.FlashAttnBwd(q, k, v, o, lse, do, BH, S, d, None, causal)
            qd, kd, vd = (t.double().requires_grad_(True) for t in (q, k, v))
            ref = F.scaled_dot_product_attention(qd, kd, vd, is_causal=causal)
            rq, rk, rv = torch.autograd.grad(ref, (qd, kd, vd), do.double())
            err = lambda a, b: float((a.double() - b).abs().max() / b.abs().max())
            ms = C.BenchFlashAttn(BH, S, d, 20, causal)
            tms = timeit(lambda: F.scaled_dot_product_attention(q[None], k[None], v[None], is_causal=causal),
                         iters=20, flush=False)
            fl = 4.0 * BH * S * S * d * (0.5 if causal else 1.0)
            _emit(bench="reference_attention", dtype="bf16", BH=BH, S=S, d=d, causal=causal, ms=ms,
                  gflops=fl / 1e9 / (ms / 1e3), torch_sdpa_ms=tms, torch_sdpa_gflops=fl / 1e9 / (tms / 1e3),
                  rel_err_out=err(o, ref.detach()), rel_err_dq=err(dq, rq), rel_err_dk=err(dk, rk),
                  rel_err_dv=err(dv, rv), reference_published_gflops_fp64=86.6 if causal else 95.4)


def bench_mha(device=None, B: int = 8, S: int = 512, E: int = 512, H: int = 8, iters: int = 10):
    """The reference's MultiHeadAttention benchmark (benchmark/mha/main.go:55-103): ``Forward``
    (differentiable) against ``ForwardFused`` (inference entry point), first their largest
    difference at (2, 64, E), causal and not, then the median wall-clock time of 10 calls at
    B = 8, S = 512, E = 512, H = 8, causal, each call synchronised as there.  bf16 on CUDA
    (the tcgen05 attention core), float64 on the CPU oracle path."""
    from .. import nn
    dev = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
    dt = torch.bfloat16 if dev.type == "cuda" else torch.float64
    torch.manual_seed(0)
    mha = nn.MultiHeadAttention(E, H).to(device=dev, dtype=dt)
    diffs = {}
    for causal in (False, True):
        x = (torch.rand(2, 64, E, device=dev) * 2 - 1).to(dt)
        ref = mha.Forward(x, x, x, causal) if hasattr(mha, "Forward") else mha(x, x, x, causal)
        fused = mha.ForwardFused(x, x, x, causal)
        diffs[causal] = float((ref.detach().double() - fused.double()).abs().max())
    xl = (torch.rand(B, S, E, device=dev) * 2 - 1).to(dt)

    def sync():
        if dev.type == "cuda":
            torch.cuda.synchronize()

    def median_ms(fn, warm):
        for _ in range(warm):
            fn()
        sync()
        ts = []
        for _ in range(iters):
            t0 = time.perf_counter()
            fn()
            sync()
            ts.append((time.perf_counter() - t0) * 1e3)
        return statistics.median(ts)

    t_fwd = median_ms(lambda: mha(xl, xl, xl, True), 2)
    t_fused = median_ms(lambda: mha.ForwardFused(xl, xl, xl, True), 3)
    _emit(bench="mha", device=dev.type, dtype=str(dt).replace("torch.", ""), B=B, S=S, E=E, H=H, causal=True,
          forward_ms=t_fwd, forward_fused_ms=t_fused, max_abs_diff_noncausal=diffs[False],
          max_abs_diff_causal=diffs[True])
    return dict(forward_ms=t_fwd, forward_fused_ms=t_fused, diffs=diffs)


def bench_resident_mlp(device=None, iters: int = 20):
    """The reference's resident-MLP benchmark (benchmark/resident/main.go:75-123): the forward pass
    of 256 x 1024 -> 1024 -> 1024 -> 1024 (three products, two ReLUs) once through the tensor
    API and once on device buffers that are uploaded once (``gonn_b200.cuda``); reports both
    times and the largest difference between the two results.  float64, as there."""
    from .. import cuda as C
    from .. import tensor as T
    dev = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
    Bn, D = 256, 1024
    g = torch.Generator().manual_seed(0)
    x = torch.randn(Bn, D, dtype=torch.float64, generator=g)
    ws = [torch.randn(D, D, dtype=torch.float64, generator=g) / 32 for _ in range(3)]

    def eager():
        h = x.to(dev)                                   # the eager path pays the upload every call
        for i, w in enumerate(ws):
            h = T.MatMul(h, w.to(dev))
            if i < 2:
                h = T.Unary(h, "relu")
        return h.cpu()

    dx = C.DevUpload(x.numpy(), device=dev)
    dws = [C.DevUpload(w.numpy(), device=dev) for w in ws]
    h1, h2 = C.DevAlloc(Bn * D, device=dev), C.DevAlloc(Bn * D, device=dev)

    def resident():
        C.DevMatMul(dx, dws[0], h1, Bn, D, D)
        C.DevReLU(h1, Bn * D)
        C.DevMatMul(h1, dws[1], h2, Bn, D, D)
        C.DevReLU(h2, Bn * D)
        C.DevMatMul(h2, dws[2], h1, Bn, D, D)

    def wall(fn):
        for _ in range(3):
            fn()
        C.DevSync()
        t0 = time.perf_counter()
        for _ in range(iters):
            fn()
        C.DevSync()
        return (time.perf_counter() - t0) * 1e3 / iters

    t_eager, t_res = wall(eager), wall(resident)
    diff = float(np_abs_max(eager().numpy().reshape(-1) - h1.Download()))
    rec = dict(bench="resident_mlp", device=dev.type, dtype="float64", eager_ms=t_eager, resident_ms=t_res,
               speedup=t_eager / t_res, max_abs_diff=diff, reference_published="10.7 ms resident vs 21.4 ms eager")
    _emit(**rec)
    return rec


def np_abs_max(a):
    import numpy as np
    return np.abs(a).max()


def bench_norm():
    """LayerNorm / RMSNorm forward and backward against the stock torch ops; bytes are the
    algorithmic ones (forward reads x and writes y; backward reads x and dy and writes dx)."""
    from ..ops.norm import layer_norm, rms_norm
    F = torch.nn.functional
    for rows, D in ((16384, 768), (65536, 768), (16384, 2048), (65536, 2048), (8192, 4096), (16384, 1024)):
        for rms in (False, True):
            x = torch.randn(rows, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
            w = torch.ones(D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
            b = None if rms else torch.zeros(D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
            ours = (lambda: rms_norm(x, w)) if rms else (lambda: layer_norm(x, w, b))
            stock = (lambda: F.rms_norm(x, (D,), w, 1e-6)) if rms else (lambda: F.layer_norm(x, (D,), w, b))
            with torch.no_grad():
                t = timeit(ours)
                r = timeit(stock)
            by = 2.0 * rows * D * 2
            name = "rms_norm" if rms else "layer_norm"
            _emit(bench=name + "_fwd", rows=rows, D=D, ms=t, gbs=by / t / 1e6, torch_ms=r, torch_gbs=by / r / 1e6)
            dy = torch.randn(rows, D, device="cuda", dtype=torch.bfloat16)
            params = (x, w) if rms else (x, w, b)
            y = ours()
            t = timeit(lambda: torch.autograd.grad(y, params, dy, retain_graph=True))
            yt = stock()
            r = timeit(lambda: torch.autograd.grad(yt, params, dy, retain_graph=True))
            by = 3.0 * rows * D * 2
            _emit(bench=name + "_bwd", rows=rows, D=D, ms=t, gbs=by / t / 1e6, torch_ms=r, torch_gbs=by / r / 1e6)


def bench_mlp_cpu():
    """MLP 784 -> 256 -> 128 -> 10, batch 64, SGD with momentum, fp64 on the CPU oracle path;
    then the same step with two data-parallel ranks over the TCP star (threads)."""
    from ..models.mlp import MLP
    from ..nn.loss import CrossEntropyLoss
    from ..optim import SGD
    torch.manual_seed(0)
    model = MLP([784, 256, 128, 10], dtype=torch.float64)
    opt = SGD(model.parameters(), lr=0.05, momentum=0.9)
    x = torch.randn(64, 784, dtype=torch.float64)
    y = torch.randint(0, 10, (64,))

    def step():
        opt.zero_grad()
        loss = CrossEntropyLoss(model(x), y)
        loss.backward()
        opt.step()
        return loss

    for _ in range(5):
        step()
    t0 = time.perf_counter()
    n = 50
    for _ in range(n):
        step()
    dt = (time.perf_counter() - t0) / n
    _emit(bench="mlp_cpu", dtype="fp64", batch=64, ms_per_step=dt * 1e3, steps_per_s=1 / dt, images_per_s=64 / dt)
    # two data-parallel ranks (processes, half the cores each), 64 images per rank, gradients averaged
    # over the TCP star every step (distributed/distributed.go:249-293, 422-428)
    import multiprocessing as mp
    from ..distributed import free_addr
    ctx = mp.get_context("spawn")
    addr, q = free_addr(), ctx.Queue()
    procs = [ctx.Process(target=_mlp_dp_rank, args=(r, 2, addr, q)) for r in range(2)]
    for p in procs:
        p.start()
    times = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(30)
    dt2 = max(times)
    _emit(bench="mlp_cpu_dp2", dtype="fp64", ranks=2, batch_per_rank=64, transport="TCP star, loopback",
          ms_per_step=dt2 * 1e3, steps_per_s=1 / dt2, images_per_s=128 / dt2)


def _mlp_dp_rank(rank: int, world: int, addr: str, q):
    """One rank of the two-process data-parallel MLP benchmark; puts its seconds per step on ``q``."""
    from .. import distributed as D
    from ..models.mlp import MLP
    from ..nn.loss import CrossEntropyLoss
    from ..optim import SGD
    torch.set_num_threads(max(1, (os.cpu_count() or 2) // world))
    torch.manual_seed(rank)
    g = D.Init(rank, world, [addr], timeout=60.0)
    try:
        model = MLP([784, 256, 128, 10], dtype=torch.float64)
        g.BroadcastParams(list(model.parameters()), 0)
        opt = SGD(model.parameters(), lr=0.05, momentum=0.9)
        x = torch.randn(64, 784, dtype=torch.float64)
        y = torch.randint(0, 10, (64,))

        def step():
            opt.zero_grad()
            CrossEntropyLoss(model(x), y).backward()
            D.DDPStep(g, opt)

        for _ in range(5):
            step()
        g.Barrier()
        t0 = time.perf_counter()
        n = 50
        for _ in range(n):
            step()
        g.Barrier()
        q.put((time.perf_counter() - t0) / n)
    finally:
        g.Close()


def bench_allreduce():
    """Bus bandwidth of the peer-memory all-reduce against NCCL: 1 KB .. 1 GB, with plain peer
    loads / stores ("p2p", fixed summation order) and through the NVSwitch multicast mapping
    ("multimem"); sizes up to 64 KiB take the one-shot kernel in both."""
    import torch.distributed as dist
    from ..distributed.nvlink import SymmetricMemory
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    max_bytes = 1 << 30
    nccl_cache = {}
    for mode in ("p2p", "multimem"):
        symm = SymmetricMemory(max_bytes, rank, world, device=torch.device("cuda", local), multicast=mode == "multimem")
        if mode == "multimem" and not symm.multicast:
            if rank == 0:
                _emit(bench="allreduce", mode=mode, unavailable="no multicast mapping: " + str(getattr(symm, "_vmm_error", None)))
            symm.close()
            continue
        for dt in (torch.bfloat16, torch.float32):
            esz = 2 if dt == torch.bfloat16 else 4
            nbytes = 1 << 10
            while nbytes <= max_bytes:
                n = nbytes // esz
                n = max(n // (world * 8) * (world * 8), world * 8)
                buf = symm.view(0, n, dt)
                buf.fill_(1.0)
                ref = torch.ones(n, device="cuda", dtype=dt)
                ctas = 8 if nbytes <= (1 << 16) else (32 if nbytes <= (1 << 22) else 128)

                def ours():
                    symm.all_reduce(0, n, dt, "mean", ctas)

                def nccl():
                    dist.all_reduce(ref, op=dist.ReduceOp.AVG)

                res = []
                for name, fn in (("ours", ours), ("nccl", nccl)):
                    if name == "nccl" and (dt, nbytes) in nccl_cache:
                        res.append(nccl_cache[(dt, nbytes)])
                        continue
                    for _ in range(3):
                        fn()
                    torch.cuda.synchronize()
                    dist.barrier()
                    iters = 20 if nbytes <= (1 << 24) else 5
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for _ in range(iters):
                        fn()
                    e1.record()
                    torch.cuda.synchronize()
                    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)   # slowest rank
                    res.append(float(t.item()))
                nccl_cache[(dt, nbytes)] = res[1]
                symm.check()
                if rank == 0:
                    bus = lambda ms: 2.0 * (world - 1) / world * n * esz / ms / 1e6
                    _emit(bench="allreduce", mode=mode, dtype=str(dt), bytes=n * esz, world=world, ms=res[0],
                          bus_gbs=bus(res[0]), nccl_ms=res[1], nccl_bus_gbs=bus(res[1]),
                          timing="back-to-back calls, max over ranks")
                nbytes *= 4
        symm.close()
    dist.destroy_process_group()


def bench_host_time():
    """Host time of one training step of the 12-layer LM: launched kernel by kernel (with the
    functions that cost the most, from cProfile) and replayed as one CUDA graph.  Host time is the
    wall-clock time of the Python call without a device synchronisation inside; the device time of
    the same steps is printed beside it."""
    import cProfile
    import io
    import pstats
    import time
    from ..distributed.ddp import DistributedDataParallel
    from ..models.lm import TransformerLM
    from ..utils.graph import GraphedStep
    dev = torch.device("cuda", 0)
    model = TransformerLM(32000, 768, 12, 12, 3072, 1024, dtype=torch.bfloat16, device=dev)
    ddp = DistributedDataParallel(model, optimizer=dict(kind="adamw", lr=3e-4, weight_decay=0.1))
    ids = torch.randint(0, 32000, (16, 1024), device=dev)
    tgt = torch.roll(ids, -1, 1)

    def step(x, y):
        loss = model.loss(x, y)
        loss.backward()
        ddp.step()
        return loss

    def host_and_device(fn, n=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        host = 0.0
        e0.record()
        for _ in range(n):
            t0 = time.perf_counter()
            fn()
            host += time.perf_counter() - t0
        e1.record()
        torch.cuda.synchronize()
        return host / n * 1e3, e0.elapsed_time(e1) / n

    h, d = host_and_device(lambda: step(ids, tgt))
    _emit(bench="host_time", mode="eager", host_ms_per_step=h, device_ms_per_step=d)
    prof = cProfile.Profile()
    prof.enable()
    for _ in range(3):
        step(ids, tgt)
    prof.disable()
    torch.cuda.synchronize()
    out = io.StringIO()
    pstats.Stats(prof, stream=out).sort_stats("tottime").print_stats(14)
    print(out.getvalue())
    graphed = GraphedStep(step, ddp, (ids, tgt), warmup=2)
    gx, gy = graphed.inputs
    h, d = host_and_device(lambda: graphed(gx, gy))
    _emit(bench="host_time", mode="cuda graph replay", host_ms_per_step=h, device_ms_per_step=d,
          kernels_per_step=graphed.launches_per_step)


def bench_secondary():
    """Operators outside the training steps, 2^26 bf16 elements (8192 x 8192): dropout, row softmax, a
    row-vector broadcast multiply, arg-max over columns, each beside torch's kernel for the same call."""
    from ..ops import elementwise as ew
    from ..ops.dropout import dropout
    from ..ops.reduce import reduce_axis
    from ..ops.softmax import softmax
    a = torch.randn(1 << 26, device="cuda", dtype=torch.bfloat16)
    m = a.view(8192, 8192)
    b = torch.randn(8192, device="cuda", dtype=torch.bfloat16)
    for name, ours, ref in (("dropout p=0.1", lambda: dropout(a, 0.1), lambda: torch.nn.functional.dropout(a, 0.1)),
                            ("softmax rows of 8192", lambda: softmax(m, -1), lambda: torch.softmax(m, -1)),
                            ("(8192 x 8192) * (8192)", lambda: ew.binary_forward("mul", m, b), lambda: m * b),
                            ("argmax over columns", lambda: reduce_axis(m, 0, "argmax"), lambda: m.argmax(0))):
        _emit(bench="secondary", op=name, us=timeit(ours) * 1e3, torch_us=timeit(ref) * 1e3)


def main(argv):
    kind = argv[0] if argv else "gemm"
    fn = {"gemm": bench_gemm, "elementwise": bench_elementwise, "flash": bench_flash, "norm": bench_norm,
          "mlp": bench_mlp_cpu, "allreduce": bench_allreduce, "refattn": bench_reference_attention, "resident": bench_resident_mlp,
          "hosttime": bench_host_time, "secondary": bench_secondary, "mha": bench_mha}.get(kind)
    if fn is None:
        raise SystemExit(f"unknown benchmark {kind!r}")
    fn()


if __name__ == "__main__":
    main(sys.argv[1:])

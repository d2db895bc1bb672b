"""Small, self-contained workloads for profiling one kernel at a time.

    python -m gonn_b200.utils.profile_cases gemm 4096 4096 4096 [nt|nn|tn] [bias_gelu|bias_res|pair]
    python -m gonn_b200.utils.profile_cases flash_fwd 4 2048 16 128 [causal]
    python -m gonn_b200.utils.profile_cases flash_bwd 4 2048 16 128 [causal]
    python -m gonn_b200.utils.profile_cases norm 16384 768
    python -m gonn_b200.utils.profile_cases norm_bwd 16384 768        # LayerNorm backward
    python -m gonn_b200.utils.profile_cases norm_fork 16384 768       # backward with the residual bypass fused
    python -m gonn_b200.utils.profile_cases step 50000000
    python -m gonn_b200.utils.profile_cases conv 256 64 128 15 15     # N C_in C_out H W, 3x3: forward + backward

Each case allocates a few hundred MB at most, runs three warm-up launches and
then five timed launches (CUDA events), and prints one line with the time and the
achieved rate.  Under ``ncu`` select the kernel with ``-k`` and skip the warm-up
launches with ``-s 3 -c 1``.
"""
from __future__ import annotations

import math
import sys

import torch


def _time(fn, iters=5):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main(argv):
    from .. import lib
    from ..ops.attention import flash_bwd, flash_fwd
    from ..ops.gemm import gemm
    from ..ops.norm import layer_norm
    kind = argv[0]
    dev = "cuda"
    if kind == "gemm":
        M, N, K = (int(a) for a in argv[1:4])
        layout = argv[4] if len(argv) > 4 else "nt"
        epi = argv[5] if len(argv) > 5 else ""
        ta, tb = layout[0] == "t", layout[1] == "t"
        a = torch.randn((K, M) if ta else (M, K), device=dev, dtype=torch.bfloat16)
        b = torch.randn((N, K) if tb else (K, N), device=dev, dtype=torch.bfloat16)
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        kw = {}
        if epi == "bias_gelu":
            kw = dict(bias=torch.randn(N, device=dev, dtype=torch.bfloat16), act="gelu",
                      aux=torch.empty(M, N, device=dev, dtype=torch.bfloat16), aux_mode="store_pre")
        elif epi == "bias_res":
            kw = dict(bias=torch.randn(N, device=dev, dtype=torch.bfloat16),
                      aux=torch.randn(M, N, device=dev, dtype=torch.bfloat16), aux_mode="add")
        elif epi == "pair":
            kw = dict(force_bn=512)  # the two-CTA (256 x 256 per SM pair) kernel
        ms = _time(lambda: gemm(a, b, trans_a=ta, trans_b=tb, out=out, **kw))
        print(f"gemm {M}x{N}x{K} {layout} {epi}: {ms:.4f} ms, {2 * M * N * K / ms / 1e9:.1f} TFLOP/s")
    elif kind in ("flash_fwd", "flash_bwd"):
        B, S, H, D = (int(a) for a in argv[1:5])
        causal = len(argv) > 5 and argv[5] == "causal"
        q, k, v = (torch.randn(B, S, H, D, device=dev, dtype=torch.bfloat16) for _ in range(3))
        scale = 1 / math.sqrt(D)
        out, lse = flash_fwd(q, k, v, causal, scale)
        fl = 4 * B * H * S * S * D * (0.5 if causal else 1.0)
        if kind == "flash_fwd":
            ms = _time(lambda: flash_fwd(q, k, v, causal, scale))
            print(f"flash_fwd B{B} S{S} H{H} D{D} causal={causal}: {ms:.4f} ms, {fl / ms / 1e9:.1f} TFLOP/s")
        else:
            do = torch.randn_like(out)
            ms = _time(lambda: flash_bwd(q, k, v, out, do, lse, causal, scale))
            print(f"flash_bwd B{B} S{S} H{H} D{D} causal={causal}: {ms:.4f} ms, {2.5 * fl / ms / 1e9:.1f} TFLOP/s "
                  "(2.5x forward FLOPs convention)")
    elif kind == "norm":
        rows, D = int(argv[1]), int(argv[2])
        x = torch.randn(rows, D, device=dev, dtype=torch.bfloat16)
        w = torch.ones(D, device=dev, dtype=torch.bfloat16)
        b = torch.zeros(D, device=dev, dtype=torch.bfloat16)
        ms = _time(lambda: layer_norm(x, w, b))
        print(f"layer_norm {rows}x{D}: {ms:.4f} ms, {2 * rows * D * 2 / ms / 1e6:.1f} GB/s")
    elif kind in ("norm_bwd", "norm_fork"):
        from ..ops.norm import norm_fork
        rows, D = int(argv[1]), int(argv[2])
        x = torch.randn(rows, D, device=dev, dtype=torch.bfloat16, requires_grad=True)
        w = torch.ones(D, device=dev, dtype=torch.bfloat16, requires_grad=True)
        b = torch.zeros(D, device=dev, dtype=torch.bfloat16, requires_grad=True)
        dy = torch.randn(rows, D, device=dev, dtype=torch.bfloat16)
        if kind == "norm_bwd":
            y = layer_norm(x, w, b)
            ms = _time(lambda: torch.autograd.grad(y, (x, w, b), dy, retain_graph=True))
            nb = 3
        else:
            rb = torch.zeros(D, device=dev, dtype=torch.bfloat16, requires_grad=True)
            y, xp = norm_fork(x, w, b, 1e-5, False, rb)
            dp = torch.randn(rows, D, device=dev, dtype=torch.bfloat16)
            ms = _time(lambda: torch.autograd.grad((y, xp), (x, w, b, rb), (dy, dp), retain_graph=True))
            nb = 4
        print(f"{kind} {rows}x{D}: {ms:.4f} ms, {nb * rows * D * 2 / ms / 1e6:.1f} GB/s")
    elif kind == "conv":
        from ..nn.conv import Conv2d
        N, Ci, Co, H, W = (int(a) for a in argv[1:6])
        conv = Conv2d(Ci, Co, 3, dtype=torch.bfloat16, device=dev)
        x = torch.randn(N, Ci, H, W, device=dev, dtype=torch.bfloat16, requires_grad=True)
        y = conv(x)
        g = torch.randn_like(y)
        ms_f = _time(lambda: conv(x))
        ms_b = _time(lambda: torch.autograd.grad(y, (x, conv.weight, conv.bias), g, retain_graph=True))
        fl = 2.0 * N * Co * Ci * 9 * (H - 2) * (W - 2)
        print(f"conv {N}x{Ci}->{Co} {H}x{W}: fwd {ms_f:.4f} ms ({fl / ms_f / 1e9:.1f} TFLOP/s), "
              f"bwd {ms_b:.4f} ms ({2 * fl / ms_b / 1e9:.1f} TFLOP/s)")
    elif kind == "step":
        n = int(argv[1]) // 8 * 8
        from ..distributed.nvlink import SymmetricMemory
        sm = SymmetricMemory(4 * n + (2 << 20))
        master = torch.randn(n, device=dev)
        m = torch.zeros(n, device=dev)
        v = torch.zeros(n, device=dev)
        hy = [1e-3, 0.1, 0.9, 0.999, 1e-8, 0.1, 0.001, 1.0]
        ms = _time(lambda: sm.fused_step(1, torch.bfloat16, 1 << 20, (1 << 20) + 2 * n, n, master, m, v, hy, 296))
        print(f"fused_step n={n}: {ms:.4f} ms, {28 * n / ms / 1e6:.1f} GB/s")
    else:
        raise SystemExit(f"unknown case {kind}")
    lib.assert_status_ok()


if __name__ == "__main__":
    main(sys.argv[1:])

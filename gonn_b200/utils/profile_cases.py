"""Small, self-contained workloads for profiling one kernel at a time.

    python -m gonn_b200.utils.profile_cases gemm 4096 4096 4096 [nt|nn|tn] [bias_gelu|bias_res|pair]
    python -m gonn_b200.utils.profile_cases flash_fwd 4 2048 16 128 [causal]
    python -m gonn_b200.utils.profile_cases flash_bwd 4 2048 16 128 [causal] [nospill]
    python -m gonn_b200.utils.profile_cases norm 16384 768
    python -m gonn_b200.utils.profile_cases norm_bwd 16384 768        # LayerNorm backward
    python -m gonn_b200.utils.profile_cases norm_fork 16384 768       # backward with the residual bypass fused
    python -m gonn_b200.utils.profile_cases step 50000000
    python -m gonn_b200.utils.profile_cases conv 256 64 128 15 15     # N C_in C_out H W, 3x3: forward + backward
    python -m gonn_b200.utils.profile_cases general_attn 4 512 8 64 [bf16|fp32|fp64] [plain]
                                                                       # B S H D: masked + dropout attention, fwd and bwd
    python -m gonn_b200.utils.profile_cases suite                      # one launch or two of every other kernel family
    python -m gonn_b200.utils.profile_cases suite2                     # ... and of the families `suite` leaves out

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
            if "nospill" in argv:          # dQ by a second pass instead of the dS^T workspace
                from ..ops import attention as _att
                _att.set_ds_spill_limit(0)
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
    elif kind == "suite":
        # Memory-bound and small kernels, each on an input of a few hundred MB at most (larger than the
        # 126 MB L2 where the kernel streams).  Every op runs twice; a profiler keeps the last launch.
        from .. import nn, optim, quant
        from ..nn.batchnorm import BatchNorm2d
        from ..ops import elementwise as ew
        from ..ops.attention import general_attention
        from ..ops.norm import norm_fork, rms_norm
        from ..ops.reduce import column_sum
        from ..ops.softmax import cross_entropy
        bf = torch.bfloat16
        for rep in range(2):
            # elementwise: binary add, unary gelu forward / backward, cast
            a = torch.randn(1 << 26, device=dev, dtype=bf)
            b = torch.randn(1 << 26, device=dev, dtype=bf)
            ew.binary_forward("add", a, b)
            g = ew.unary_forward("gelu", a)
            ew.unary_backward("gelu", a, b)
            a.float()
            del a, b, g
            # norms: LayerNorm forward / backward / fork backward, RMSNorm forward
            x = torch.randn(65536, 768, device=dev, dtype=bf, requires_grad=True)
            w = torch.ones(768, device=dev, dtype=bf, requires_grad=True)
            bb = torch.zeros(768, device=dev, dtype=bf, requires_grad=True)
            rb = torch.zeros(768, device=dev, dtype=bf, requires_grad=True)
            dy = torch.randn(65536, 768, device=dev, dtype=bf)
            torch.autograd.grad(layer_norm(x, w, bb), (x, w, bb), dy)
            y, xp = norm_fork(x, w, bb, 1e-5, False, rb)
            torch.autograd.grad((y, xp), (x, w, bb, rb), (dy, dy))
            rms_norm(x.detach(), w.detach())
            column_sum(dy)
            del x, dy, y, xp
            # softmax cross-entropy forward + in-place backward on LM-sized logits
            logits = torch.randn(8192, 32000, device=dev, dtype=bf, requires_grad=True)
            tgt = torch.randint(0, 32000, (8192,), device=dev)
            cross_entropy(logits, tgt).backward()
            del logits
            # embedding gather and deterministic scatter-add backward
            emb = nn.Embedding(32000, 768, dtype=bf, device=dev)
            ids = torch.randint(0, 32000, (16, 1024), device=dev)
            emb(ids).sum().backward()
            # BatchNorm forward / backward, max pooling forward / backward
            bn = BatchNorm2d(64, dtype=bf, device=dev)
            img = torch.randn(256, 64, 30, 30, device=dev, dtype=bf, requires_grad=True)
            pool = nn.MaxPool2d(2)
            pool(bn(img)).sum().backward()
            # int8 Linear (dynamic quantisation: observe, quantise, int8 tcgen05 GEMM with dequantising epilogue)
            lin = nn.Linear(4096, 4096, dtype=torch.float32, device=dev)
            ql = quant.NewDynamicLinearFrom(lin)
            ql(torch.randn(8192, 4096, device=dev))
            # multi-tensor AdamW over a few dozen tensors and global-norm clipping
            ps = [torch.nn.Parameter(torch.randn(1024, 1024, device=dev)) for _ in range(32)]
            for p_ in ps:
                p_.grad = torch.randn_like(p_)
            opt = optim.AdamW(ps, lr=1e-3)
            optim.ClipGradNorm(ps, 1.0)
            opt.step()
            del ps, opt
            # exact-precision GEMMs: fp64 tensor-core kernel, fp32 as three bf16 planes (split + tcgen05)
            a64 = torch.randn(2048, 2048, device=dev, dtype=torch.float64)
            gemm(a64, a64)
            a32 = torch.randn(2048, 2048, device=dev)
            gemm(a32, a32)
            # split-K weight-gradient GEMM with its finish kernel
            dyw = torch.randn(16384, 768, device=dev, dtype=bf)
            xw = torch.randn(16384, 3072, device=dev, dtype=bf)
            gemm(dyw, xw, trans_a=True)
            # general attention (masked, dropout), forward and backward
            q = torch.randn(4, 512, 8, 64, device=dev, dtype=bf, requires_grad=True)
            kk = torch.randn(4, 512, 8, 64, device=dev, dtype=bf, requires_grad=True)
            vv = torch.randn(4, 512, 8, 64, device=dev, dtype=bf, requires_grad=True)
            mask = torch.rand(512, 512, device=dev) < 0.2
            general_attention(q, kk, vv, True, None, mask, None, 0.1, 7).sum().backward()
            torch.cuda.synchronize()
        print("suite done")
    elif kind == "general_attn":
        # The SIMT attention kernel: causal + boolean mask + dropout 0.1 (or none of the three with `plain`).
        from ..ops.attention import general_attention
        B, S, H, D = (int(a) for a in argv[1:5])
        dt = {"bf16": torch.bfloat16, "fp32": torch.float32, "fp64": torch.float64}[argv[5] if len(argv) > 5 else "bf16"]
        plain = "plain" in argv
        q, kk, vv = (torch.randn(B, S, H, D, device=dev, dtype=dt, requires_grad=True) for _ in range(3))
        mask = None if plain else torch.rand(S, S, device=dev) < 0.2
        p = 0.0 if plain else 0.1

        def fwd():
            with torch.no_grad():
                return general_attention(q, kk, vv, not plain, None, mask, None, p, 7)

        def fwd_bwd():
            q.grad = kk.grad = vv.grad = None
            general_attention(q, kk, vv, not plain, None, mask, None, p, 7).sum().backward()

        fl = 4 * B * H * S * S * D
        tf = _time(fwd)
        tb = _time(fwd_bwd)
        print(f"general_attn B{B} S{S} H{H} D{D} {dt} plain={plain}: forward {tf:.4f} ms ({fl / tf / 1e9:.2f} TFLOP/s of "
              f"the full square), forward + backward {tb:.4f} ms")
    elif kind == "suite2":
        # The kernel families that neither the training steps nor `suite` launch: recurrent gates, dropout,
        # casts, scans, transposes, standalone softmax, fake quantisation, row / column reductions with
        # arg-max, broadcasting binary ops, the gather / scatter convolution path, overlapping pooling,
        # the consuming cross-entropy and the attention backward with its dS^T product.
        from .. import nn, quant
        from ..ops import elementwise as ew
        from ..ops.dropout import dropout
        from ..ops.reduce import reduce_axis
        from ..ops.shape import cumsum, transpose_last2
        from ..ops.softmax import cross_entropy, log_softmax, softmax
        bf = torch.bfloat16
        for rep in range(2):
            seq = torch.randn(64, 32, 512, device=dev, dtype=bf, requires_grad=True)
            for cell in (nn.LSTM(512, 512, dtype=bf, device=dev), nn.GRU(512, 512, dtype=bf, device=dev)):
                cell(seq).sum().backward()
            a = torch.randn(1 << 26, device=dev, dtype=bf, requires_grad=True)
            dropout(a, 0.1).sum().backward()
            ew.cast(a.detach(), torch.float32)
            ew.binary_forward("mul", a.detach().view(8192, 8192), torch.randn(8192, device=dev, dtype=bf))
            del a
            m = torch.randn(8192, 8192, device=dev, dtype=bf, requires_grad=True)
            transpose_last2(m.detach())
            cumsum(m.detach().float(), -1)
            softmax(m, -1).sum().backward()
            log_softmax(m.detach(), -1)
            reduce_axis(m.detach(), 1, "sum"); reduce_axis(m.detach(), 1, "argmax"); reduce_axis(m.detach(), 0, "argmax")
            reduce_axis(m.detach().float(), 0, "max")
            fq = quant.FakeQuant()
            fq(m.float()).sum().backward()
            del m
            img = torch.randn(64, 32, 64, 64, device=dev, dtype=bf, requires_grad=True)
            conv = nn.Conv2d(32, 64, 3, padding=1, dilation=2, groups=2, dtype=bf, device=dev)   # gather + GEMM path
            nn.MaxPool2d(3, 2, 1)(conv(img)).sum().backward()                                     # overlapping windows
            lg = torch.randn(8192, 32000, device=dev, dtype=bf, requires_grad=True)
            cross_entropy(lg * 1, torch.randint(0, 32000, (8192,), device=dev), inplace_backward=True,
                          consume_logits=True).backward()
            del lg
            q, k, v = (torch.randn(16, 1024, 12, 64, device=dev, dtype=bf) for _ in range(3))
            o, lse = flash_fwd(q, k, v, True, 0.125)
            flash_bwd(q, k, v, o, torch.randn_like(o), lse, True, 0.125)
            torch.cuda.synchronize()
        print("suite2 done")
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

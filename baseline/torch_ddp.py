"""NCCL + cuBLAS baseline: the same models written with stock PyTorch layers, trained with
torch DDP, torch's fused AdamW and bf16 autocast over fp32 parameters (the usual PyTorch
recipe), or with ``--twin bf16`` entirely in bf16 (bf16 parameters, no cast kernels, no fp32
copy of the logits): the faster of the two is the number to compare against.  Prints the same
JSON line as bench.py with "impl": "torch-ddp".

    python baseline/torch_ddp.py --config lm --steps 10 --warmup 3
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 baseline/torch_ddp.py --gpus 8
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F


class Block(nn.Module):
    def __init__(self, d, h, ff, rms=False):
        super().__init__()
        self.h = h
        self.n1 = nn.RMSNorm(d, eps=1e-6) if rms else nn.LayerNorm(d)
        self.n2 = nn.RMSNorm(d, eps=1e-6) if rms else nn.LayerNorm(d)
        self.qkv = nn.Linear(d, 3 * d)
        self.o = nn.Linear(d, d)
        self.f1 = nn.Linear(d, ff)
        self.f2 = nn.Linear(ff, d)

    def forward(self, x):
        B, S, D = x.shape
        q, k, v = self.qkv(self.n1(x)).view(B, S, 3, self.h, D // self.h).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, S, D)
        x = x + self.o(a)
        return x + self.f2(F.gelu(self.f1(self.n2(x)), approximate="tanh"))


class LM(nn.Module):
    def __init__(self, vocab, d, layers, heads, ff, max_seq, rms=False):
        super().__init__()
        self.tok, self.pos = nn.Embedding(vocab, d), nn.Embedding(max_seq, d)
        self.layers = nn.ModuleList([Block(d, heads, ff, rms) for _ in range(layers)])
        self.norm = nn.RMSNorm(d, eps=1e-6) if rms else nn.LayerNorm(d)
        self.head = nn.Linear(d, vocab, bias=False)

    def forward(self, ids):
        x = self.tok(ids) + self.pos(torch.arange(ids.shape[1], device=ids.device))[None]
        for l in self.layers:
            x = l(x)
        return self.head(self.norm(x))


class CNN(nn.Module):
    """conv3x3(3->64) - BN - ReLU - maxpool2 - conv3x3(64->128) - BN - ReLU - global average - linear."""

    def __init__(self):
        super().__init__()
        self.c1, self.b1 = nn.Conv2d(3, 64, 3), nn.BatchNorm2d(64)
        self.c2, self.b2 = nn.Conv2d(64, 128, 3), nn.BatchNorm2d(128)
        self.fc = nn.Linear(128, 10)

    def forward(self, x):
        x = F.max_pool2d(F.relu(self.b1(self.c1(x))), 2)
        x = F.relu(self.b2(self.c2(x))).mean((2, 3))
        return self.fc(x)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--config", default="lm", choices=["lm", "gpt", "cnn"])
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--twin", default="autocast", choices=["autocast", "bf16"],
                    help="autocast: fp32 parameters under torch.autocast with fp32 logits into the loss (torch's "
                         "documented mixed-precision recipe); bf16: parameters, activations and logits all bf16, no "
                         "cast kernels, fused AdamW on the bf16 parameters (the fastest plain-torch build of the model)")
    a = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    lr = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(1234)
    if a.config == "cnn":
        model, B, S, V = CNN().to(dev).to(memory_format=torch.channels_last), a.batch or 256, 1, 10
        if world > 1:
            model = nn.SyncBatchNorm.convert_sync_batchnorm(model)
    elif a.config == "lm":
        model, B, S, V = LM(32000, 768, 12, 12, 3072, 1024).to(dev), a.batch or 16, 1024, 32000
    else:
        model, B, S, V = LM(50304, 2048, 24, 16, 8192, 2048, rms=True).to(dev), a.batch or 4, 2048, 50304
    pure = a.twin == "bf16"
    if pure:
        model = model.to(torch.bfloat16)
    net = nn.parallel.DistributedDataParallel(model, device_ids=[lr], gradient_as_bucket_view=True) if world > 1 else model
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, weight_decay=0.1, fused=True)
    g = torch.Generator().manual_seed(100 + rank)
    if a.config == "cnn":
        x = torch.randn(B, 3, 32, 32, generator=g).to(dev).contiguous(memory_format=torch.channels_last)
        if pure:
            x = x.to(torch.bfloat16)
        y = torch.randint(0, 10, (B,), generator=g).to(dev)
    else:
        x = torch.randint(0, V, (B, S), generator=g).to(dev)
        y = torch.roll(x, -1, 1)

    def step():
        if pure:
            loss = F.cross_entropy(net(x).view(-1, V), y.view(-1))
        else:
            with torch.autocast("cuda", dtype=torch.bfloat16):
                logits = net(x)
            loss = F.cross_entropy(logits.view(-1, V).float(), y.view(-1))
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)

    for _ in range(a.warmup):
        step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        step()
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(json.dumps({"impl": "torch-ddp", "metric": "training throughput", "config": a.config,
                          "value": B * S * world * a.steps / (ms.item() / 1e3), "unit": "images/s" if a.config == "cnn" else "tokens/s", "n_gpus": world,
                          "ms_per_step": ms.item() / a.steps, "steps": a.steps, "warmup": a.warmup, "twin": a.twin,
                          "dtype": "bf16 parameters and activations" if pure else "bf16 autocast over fp32 parameters"}))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

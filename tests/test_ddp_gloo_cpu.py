"""The data-parallel engine on two CPU ranks (gloo): bucket bookkeeping, gradient sinks and
hooks, the sharded AdamW state and the parameter all-gather run exactly as on GPUs, with the
collectives carried by torch.distributed instead of the peer-memory kernels."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

LM = dict(vocab=48, d_model=32, n_layers=2, n_heads=2, d_ff=64, max_seq=12, dtype=torch.bfloat16)
OPT = dict(kind="adamw", lr=1e-2, weight_decay=0.1)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _data():
    ids = torch.randint(0, 48, (4, 12), generator=torch.Generator().manual_seed(7))
    x = torch.randn(8, 6, generator=torch.Generator().manual_seed(9))
    y = torch.randn(8, 3, generator=torch.Generator().manual_seed(10))
    return ids, x, y


def _mlp():
    from gonn_b200 import nn
    torch.manual_seed(5)
    return nn.Sequential(nn.Linear(6, 8), nn.Tanh(), nn.Linear(8, 3))


def _named(module):
    return {n: p.detach().float().clone() for n, p in module.named_parameters()}


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from gonn_b200 import optim
        from gonn_b200.distributed.ddp import DistributedDataParallel
        from gonn_b200.models.lm import TransformerLM
        ids, x, y = _data()
        torch.manual_seed(100 + rank)                      # ranks start from different values
        model = TransformerLM(**LM)
        ddp = DistributedDataParallel(model, optimizer=OPT, bucket_mb=0.01)
        res = {"buckets": len(ddp.buckets), "state_bytes": ddp.state_bytes_per_rank(),
               "master_len": [b.master.numel() for b in ddp.buckets], "bucket_len": [b.length for b in ddp.buckets],
               "init": _named(model)}                      # after the broadcast from rank 0
        mine = ids[rank * 2:(rank + 1) * 2]
        losses = []
        for _ in range(3):
            loss = model.loss(mine, mine)
            loss.backward()
            ddp.step()
            losses.append(float(loss))
        res["params"], res["losses"] = _named(model), losses
        # accumulation without communication, then one synchronised step
        with ddp.no_sync():
            model.loss(mine, mine).backward()
        model.loss(mine, mine).backward()
        ddp.step()
        res["after_accum"] = _named(model)
        # all-reduce mode: fp32 parameters, the caller's optimizer
        lin = _mlp()
        d2 = DistributedDataParallel(lin, optimizer=None, bucket_mb=0.0001)
        opt = optim.SGD(lin.parameters(), lr=0.1, momentum=0.9)
        sl = slice(rank * 4, (rank + 1) * 4)
        for _ in range(3):
            opt.zero_grad()
            ((lin(x[sl]) - y[sl]) ** 2).mean().backward()
            d2.step()
            opt.step()
        res["lin"], res["lin_buckets"] = _named(lin), len(d2.buckets)
        # a layer that only rank 0 uses: its gradients never arrive on rank 1, so the ranks see
        # their buckets complete in different orders; the collectives must still pair up
        from gonn_b200 import nn
        torch.manual_seed(11)
        br = nn.Sequential(nn.Linear(6, 6), nn.Linear(6, 6), nn.Linear(6, 3))
        d3 = DistributedDataParallel(br, optimizer=None, bucket_mb=0.00001)
        h = br[0](x[sl])
        if rank == 0:
            h = br[1](h)
        ((br[2](h) - y[sl]) ** 2).mean().backward()
        d3.step()
        res["branch_grads"] = {n: p.grad.detach().clone() for n, p in br.named_parameters()}
        res["branch_buckets"] = len(d3.buckets)
        out[rank] = res
    finally:
        dist.destroy_process_group()


def _same(a, b):
    return a.keys() == b.keys() and all(torch.equal(a[k], b[k]) for k in a)


@pytest.mark.timeout(300)
def test_two_cpu_ranks_run_the_engine():
    world, port = 2, _free_port()
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
        r0, r1 = out[0], out[1]
    # every rank starts from rank 0's values and ends every step with identical bytes
    assert _same(r0["init"], r1["init"]) and _same(r0["params"], r1["params"])
    assert _same(r0["after_accum"], r1["after_accum"]) and not _same(r0["params"], r0["after_accum"])
    assert r0["buckets"] > 2 and r0["lin_buckets"] > 1
    # ZeRO-1: each rank holds fp32 master / m / v for half of every bucket
    assert r0["master_len"] == [n // 2 for n in r0["bucket_len"]]
    assert r0["state_bytes"] == sum(3 * 4 * (n // 2) for n in r0["bucket_len"])
    assert r0["losses"][-1] < r0["losses"][0] and r1["losses"][-1] < r1["losses"][0]

    from gonn_b200 import optim
    from gonn_b200.distributed.ddp import DistributedDataParallel
    from gonn_b200.models.lm import TransformerLM
    ids, x, y = _data()
    # the same three steps in one process on the full batch (mean of the two shard losses)
    torch.manual_seed(100)
    model = TransformerLM(**LM)
    ddp = DistributedDataParallel(model, optimizer=OPT, bucket_mb=0.01, rank=0, world=1)
    assert _same(_named(model), r0["init"])
    for _ in range(3):
        (0.5 * model.loss(ids[:2], ids[:2]) + 0.5 * model.loss(ids[2:], ids[2:])).backward()
        ddp.step()
    for n, p in _named(model).items():
        assert (p - r0["params"][n]).abs().max().item() < 3e-2, n      # bf16 parameters, three AdamW steps
    # all-reduce mode, fp32: equals full-batch SGD with momentum to rounding error
    lin = _mlp()
    opt = optim.SGD(lin.parameters(), lr=0.1, momentum=0.9)
    for _ in range(3):
        opt.zero_grad()
        ((lin(x) - y) ** 2).mean().backward()
        opt.step()
    assert _same(r0["lin"], r1["lin"])
    for n, p in _named(lin).items():
        assert torch.allclose(p, r0["lin"][n], rtol=1e-5, atol=1e-6), n
    # the branch case: identical bytes on both ranks, equal to the mean of the two ranks' local
    # gradients with zeros where rank 1 had none
    from gonn_b200 import nn
    assert r0["branch_buckets"] >= 4 and _same(r0["branch_grads"], r1["branch_grads"])
    want = None
    for rank in (0, 1):
        torch.manual_seed(11)
        br = nn.Sequential(nn.Linear(6, 6), nn.Linear(6, 6), nn.Linear(6, 3))
        sl = slice(rank * 4, (rank + 1) * 4)
        h = br[0](x[sl])
        if rank == 0:
            h = br[1](h)
        ((br[2](h) - y[sl]) ** 2).mean().backward()
        g = {n: (p.grad if p.grad is not None else torch.zeros_like(p)) * 0.5 for n, p in br.named_parameters()}
        want = g if want is None else {n: want[n] + g[n] for n in g}
    for n, g in want.items():
        assert torch.allclose(g, r0["branch_grads"][n], rtol=1e-5, atol=1e-6), n

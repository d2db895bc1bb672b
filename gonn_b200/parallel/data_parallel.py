"""In-process data parallelism over shared parameters (nn/parallel/parallel.go:81-188).

``DataParallel(workers).step(opt, loss_fn, *batch)`` splits dim 0 of every batch tensor into
near-equal shards, runs ``loss_fn(*shard) * (n_k / N)`` and its backward once per shard so
that the shard gradients sum into the shared parameters, then steps the optimizer once —
the result equals one full-batch step with a mean loss.  The reference runs the shards on
goroutines and serialises leaf accumulation with a mutex; here shards on a CUDA device run
on separate streams (one per worker) and the accumulation order is fixed, shard by shard.

Caveats kept from the reference: BatchNorm sees per-shard statistics and Dropout draws per
shard, so such models do not match the single-batch run exactly.
"""
from __future__ import annotations

from typing import Callable, List, Sequence, Tuple

import torch


def shard_bounds(n: int, workers: int) -> List[Tuple[int, int]]:
    """Near-equal contiguous shards: the first ``n % workers`` shards get one extra row."""
    workers = max(1, min(workers, n))
    base, extra = divmod(n, workers)
    out, lo = [], 0
    for k in range(workers):
        hi = lo + base + (1 if k < extra else 0)
        out.append((lo, hi))
        lo = hi
    return out


def Gradients(loss_fn: Callable[..., torch.Tensor], batch: Sequence[torch.Tensor], workers: int) -> float:
    """Accumulates the gradient of the full-batch mean loss, shard by shard; returns that loss."""
    N = batch[0].shape[0]
    total = 0.0
    bounds = shard_bounds(N, workers)
    streams = None
    if batch[0].is_cuda and len(bounds) > 1:
        streams = [torch.cuda.Stream() for _ in bounds]
        for s in streams:
            s.wait_stream(torch.cuda.current_stream())
    losses = []
    for k, (lo, hi) in enumerate(bounds):
        shard = [t[lo:hi] for t in batch]
        if streams is not None:
            # forward of the shards may overlap; the backward passes below run in shard order
            with torch.cuda.stream(streams[k]):
                losses.append(loss_fn(*shard) * ((hi - lo) / N))
        else:
            losses.append(loss_fn(*shard) * ((hi - lo) / N))
    for k, l in enumerate(losses):
        if streams is not None:
            torch.cuda.current_stream().wait_stream(streams[k])
        l.backward()
        total += float(l.detach())
    return total


class DataParallel:
    def __init__(self, workers: int = 2):
        self.Workers = workers

    def step(self, opt, loss_fn: Callable[..., torch.Tensor], *batch: torch.Tensor) -> float:
        opt.zero_grad()
        loss = Gradients(loss_fn, batch, self.Workers)
        opt.step()
        return loss

    Step = step

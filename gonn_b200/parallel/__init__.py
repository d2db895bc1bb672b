"""Parallel training strategies: in-process DataParallel (nn/parallel) and re-exports of the
multi-process data-parallel engine."""
from .data_parallel import DataParallel, Gradients, shard_bounds  # noqa


def __getattr__(name):
    if name in ("DistributedDataParallel", "SymmetricMemory"):
        from .. import distributed
        return getattr(distributed, name)
    raise AttributeError(name)

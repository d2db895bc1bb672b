"""Scale-out: CPU TCP group (wire-compatible star), NVLink peer-memory collectives,
the data-parallel engine with the fused sharded-AdamW step, SyncBatchNorm."""
from .tcp import (Group, Init, DDPStep, free_addr, DistributedError, PeerTimeout, PeerClosed,  # noqa
                  ProtocolError, GroupClosed)
from . import tcp  # noqa


def __getattr__(name):
    # GPU pieces import lazily so that CPU-only use never touches CUDA
    if name in ("DistributedDataParallel", "ordered_parameters"):
        from . import ddp
        return getattr(ddp, name)
    if name in ("SymmetricMemory", "CollectiveTimeout"):
        from . import nvlink
        return getattr(nvlink, name)
    if name in ("SyncBatchNorm", "SyncBatchNorm1d", "SyncBatchNorm2d", "SyncBatchNorm3d",
                "NewSyncBatchNorm1d", "NewSyncBatchNorm2d", "NewSyncBatchNorm3d", "convert_sync_batchnorm"):
        from . import syncbn
        return getattr(syncbn, name)
    raise AttributeError(name)

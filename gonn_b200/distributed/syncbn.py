"""SyncBatchNorm: batch statistics over all ranks (distributed/syncbn.go:89-294).

Same parameters, buffers and defaults as BatchNorm (names ``weight``, ``bias``,
``running_mean``, ``running_var``).  Training forward sums [sum x | sum x^2 | count] over
the ranks, backward sums [sum dy | sum dy*xhat] while the weight / bias gradients keep the
LOCAL sums (the data-parallel wrapper averages them).  Evaluation uses the running
statistics and performs no communication.

On CUDA the exchange happens inside the normalise kernels through the symmetric peer
memory (one-shot: every rank stores its vector into every peer's slot, then sums the
slots in rank order).  On CPU ranks the sums travel through the TCP group.
"""
from __future__ import annotations

import torch

from ..nn.batchnorm import _BatchNormNd


class DeviceSync:
    """Handle to the exchange area the fused kernels use (offset inside the symmetric buffer)."""

    def __init__(self, symm, offset_bytes: int = 0):
        self.symm = symm
        self.slot_offset = symm.abs_offset(offset_bytes)


class SyncBatchNorm(_BatchNormNd):
    ranks = (2, 3, 4, 5)

    def __init__(self, num_features, eps=1e-5, momentum=0.1, affine=True, group=None, fused_relu=False, *,
                 dtype=torch.float32, device=None):
        super().__init__(num_features, eps, momentum, affine, fused_relu, dtype=dtype, device=device)
        self.group = group          # host group (TCP) or None
        self._dev_sync = None

    def attach(self, symm, offset_bytes: int = 0):
        """Uses ``symm`` (this process's symmetric memory) for the device-side exchange."""
        self._dev_sync = DeviceSync(symm, offset_bytes)
        return self

    def _sync(self):
        if self.group is not None:
            return None, self.group
        if self._dev_sync is None:
            from . import nvlink
            cur = nvlink.current()
            if cur is not None and not cur.host and cur.world > 1 and not cur.emulate:
                self._dev_sync = DeviceSync(cur, 0)
        return self._dev_sync, None


class SyncBatchNorm1d(SyncBatchNorm):
    ranks = (2, 3)


class SyncBatchNorm2d(SyncBatchNorm):
    ranks = (4,)


class SyncBatchNorm3d(SyncBatchNorm):
    ranks = (5,)


def NewSyncBatchNorm1d(group, num_features, **kw):
    return SyncBatchNorm1d(num_features, group=group, **kw)


def NewSyncBatchNorm2d(group, num_features, **kw):
    return SyncBatchNorm2d(num_features, group=group, **kw)


def NewSyncBatchNorm3d(group, num_features, **kw):
    return SyncBatchNorm3d(num_features, group=group, **kw)


def convert_sync_batchnorm(module: torch.nn.Module, group=None) -> torch.nn.Module:
    """Replaces every BatchNorm layer by a SyncBatchNorm with the same parameters and buffers."""
    for name, child in list(module.named_children()):
        if isinstance(child, _BatchNormNd) and not isinstance(child, SyncBatchNorm):
            sb = SyncBatchNorm(child.num_features, child.eps, child.momentum, child.weight is not None, group,
                               child.fused_relu, dtype=child.running_mean.dtype)
            sb.ranks = child.ranks
            sb.weight, sb.bias = child.weight, child.bias
            sb.running_mean, sb.running_var = child.running_mean, child.running_var
            sb.train(child.training)
            setattr(module, name, sb)
        else:
            convert_sync_batchnorm(child, group)
    return module

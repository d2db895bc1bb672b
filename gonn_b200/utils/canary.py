"""Canary-padded device buffers: a stand-in for a memory checker in tests.

``guarded(shape, dtype)`` carves the tensor out of the middle of a larger allocation whose
first and last ``GUARD`` bytes hold a fixed byte pattern.  A kernel that stores before the
start or past the end of the tensor (an off-by-one tile edge, a vector store that ignores a
ragged tail) lands in a guard zone instead of in a neighbour's memory, and ``Guarded.check()``
finds the changed bytes and says where.  Reads out of range cannot be caught this way; the
bounds-checked build (``python -m gonn_b200.build --debug``) covers those for the kernels
that index through tables.

    out = guarded((M, N), torch.bfloat16)
    gemm(a, b, out=out.t)
    out.check()          # raises AssertionError naming the first overwritten guard byte
"""
from __future__ import annotations

import math
from typing import Sequence

import torch

GUARD = 4096          # bytes on each side; a multiple of every alignment the kernels ask for
PATTERN = 0xA5


class Guarded:
    """A tensor ``t`` of the requested shape with guard zones on both sides."""

    def __init__(self, shape: Sequence[int], dtype: torch.dtype, device="cuda", fill=None, misalign: int = 0):
        esz = torch.empty((), dtype=dtype).element_size()
        n = int(math.prod(shape))
        if misalign % esz:
            raise ValueError("misalign must be a multiple of the element size")
        # the payload starts `misalign` bytes after a 4 KiB boundary (0 keeps it 16-byte aligned)
        body = (n * esz + misalign + 15) // 16 * 16
        self.raw = torch.full((GUARD + body + GUARD,), PATTERN, dtype=torch.uint8, device=device)
        self._lo, self._hi = GUARD + misalign, GUARD + misalign + n * esz
        self.t = self.raw[self._lo:self._hi].view(dtype).view(*shape)
        if fill is not None:
            self.t.fill_(fill)

    def check(self, what: str = "buffer") -> None:
        """Raises if any byte outside the tensor changed."""
        torch.cuda.synchronize(self.raw.device) if self.raw.is_cuda else None
        front, back = self.raw[:self._lo], self.raw[self._hi:]
        for name, zone, base in (("before", front, -self._lo), ("after", back, 0)):
            bad = (zone != PATTERN).nonzero()
            if bad.numel():
                first = int(bad[0])
                where = base + first if name == "before" else first
                raise AssertionError(f"{what}: {bad.numel()} guard bytes overwritten {name} the tensor, "
                                     f"first at byte offset {where} relative to its {'start' if name == 'before' else 'end'}")


def guarded(shape, dtype, device="cuda", fill=None, misalign: int = 0) -> Guarded:
    return Guarded(shape, dtype, device, fill, misalign)

"""Symmetric peer memory and the in-kernel collectives built on it.

What the reference does over a TCP star on the host (distributed/distributed.go:249-293 mean of the
gradients, :303-333 sum of a short vector, :338-388 parameter broadcast, :392-416 barrier, :422-428
all-reduce then optimizer step) happens here inside kernels that address the peers' memory.

``SymmetricMemory`` owns this rank's buffer (flag area + data), exchanges CUDA IPC
handles over an existing ``torch.distributed`` process group (used only as the
bootstrap channel) and exposes torch views of the local data region.  The
collectives themselves are the kernels of ``csrc/comm.cu``: they read and write
the peers' buffers directly over NVLink.

``multicast=True`` (or ``GB_COMM_MULTIMEM=1``) maps the buffers through torch's
symmetric-memory allocator instead, which also provides an NVSwitch multicast mapping; the
fused step then reduces with ``multimem.ld_reduce`` and broadcasts with ``multimem.st``
(the switch adds / replicates; each GPU moves 1/W of the plain peer traffic).  The
in-switch sum has no fixed rank order, so the default stays the plain peer path, whose
results are bit-reproducible.  Short vectors are all-reduced by a one-shot kernel (one
barrier) through a private slot area behind the data region.

With ``world == 1`` no IPC is involved; with ``emulate=W`` the W "ranks" are W
buffers on one GPU driven by a single cooperative launch (for tests).
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional

import torch

from .. import lib as _l


class _Raw:
    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 2}


class CollectiveTimeout(RuntimeError):
    """A peer did not reach a collective within the kernel's wait budget."""


_current = [None]


def current():
    """The process's symmetric memory (the native communicator is one per process), or None."""
    return _current[0]


def _apply_env_tuning():
    """``GB_STEP_INTERLEAVE`` = 0 / 1 overrides the work mapping of the fused step kernel."""
    v = os.environ.get("GB_STEP_INTERLEAVE")
    if v is not None and _l.available():
        _l.lib().gb_comm_tune(int(v))


class SymmetricMemory:
    """This rank's symmetric buffer.  Offsets handed to kernels count from the buffer's
    base (the flag area comes first); ``view`` takes offsets into the data region."""

    ONESHOT_BYTES = 2 << 20      # slot area of the one-shot all-reduce: 2 sets x world slots

    def __init__(self, data_bytes: int, rank: int = 0, world: int = 1, process_group=None,
                 emulate: int = 0, device: Optional[torch.device] = None, multicast: Optional[bool] = None):
        _apply_env_tuning()
        self.rank, self.world, self.emulate = rank, world, emulate
        _current[0] = self
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device())
        self.device = device
        self.user_bytes = (int(data_bytes) + 255) // 256 * 256
        # the one-shot slots live behind the caller's data, inside the same symmetric buffer
        self.data_bytes = self.user_bytes + (self.ONESHOT_BYTES if device.type == "cuda" else 0)
        self.multicast = False
        self._symm_handle = None
        if multicast is None:
            multicast = os.environ.get("GB_COMM_MULTIMEM", "0") == "1"
        self._raw: List[torch.Tensor] = []
        self.host = device.type != "cuda"
        self._pg = process_group
        if self.host:
            # oracle path: host memory, the collectives evaluated with tensor math; several
            # ranks exchange through torch.distributed (a CPU backend such as gloo), which
            # exercises the bucket bookkeeping and the sharded update without GPUs
            if emulate:
                raise ValueError("SymmetricMemory on the host does not emulate ranks")
            if world != 1:
                import torch.distributed as dist
                if not (dist.is_available() and dist.is_initialized()):
                    raise ValueError("SymmetricMemory on the host with several ranks needs an "
                                     "initialised torch.distributed process group (gloo)")
            self.flag_bytes = 0
            self._raw.append(torch.zeros(self.data_bytes, dtype=torch.uint8))
            return
        L = _l.lib()
        L.gb_comm_flag_bytes.restype = _l.L
        self.flag_bytes = int(L.gb_comm_flag_bytes())
        if emulate:
            self.world = emulate
            for _ in range(emulate):
                t = torch.zeros(self.flag_bytes + self.data_bytes, dtype=torch.uint8, device=self.device)
                self._raw.append(t)
            arr = (ctypes.c_void_p * emulate)(*[t.data_ptr() for t in self._raw])
            _l.call("gb_comm_emulate", _l.I(emulate), arr)
        elif world == 1:
            t = torch.zeros(self.flag_bytes + self.data_bytes, dtype=torch.uint8, device=self.device)
            self._raw.append(t)
            arr = (ctypes.c_void_p * 1)(t.data_ptr())
            _l.call("gb_comm_emulate", _l.I(1), arr)
        elif multicast and self._attach_vmm(process_group):
            pass
        else:
            import torch.distributed as dist
            base = ctypes.c_void_p()
            handle = (ctypes.c_ubyte * 64)()
            _l.call("gb_comm_alloc", _l.L(self.data_bytes), ctypes.byref(base), handle)
            handles = [None] * world
            dist.all_gather_object(handles, bytes(handle), group=process_group)
            blob = b"".join(handles)
            _l.call("gb_comm_open", _l.I(rank), _l.I(world), ctypes.c_char_p(blob))
            self._ipc = True
            self._raw.append(torch.as_tensor(_Raw(base.value, self.flag_bytes + self.data_bytes),
                                             device=self.device))
            self._raw[0][self.flag_bytes:].zero_()
            torch.cuda.synchronize()
            dist.barrier(group=process_group)

    def _attach_vmm(self, process_group) -> bool:
        """Maps the buffers through torch's symmetric-memory allocator (virtual-memory API with
        an NVSwitch multicast object where the fabric supports it).  Returns False, leaving
        nothing behind, when that allocator is unavailable; the caller then uses CUDA IPC."""
        import torch.distributed as dist
        try:
            import torch.distributed._symmetric_memory as symm
            total = self.flag_bytes + self.data_bytes
            t = symm.empty(total, dtype=torch.uint8, device=self.device)
            group = process_group if process_group is not None else dist.group.WORLD
            hdl = symm.rendezvous(t, group)
        except Exception as e:  # noqa: BLE001 - any failure of the optional path means "use IPC"
            self._vmm_error = repr(e)
            return False
        t.zero_()
        torch.cuda.synchronize()
        ptrs = [int(p) for p in hdl.buffer_ptrs]
        mc = int(getattr(hdl, "multicast_ptr", 0) or 0)        # 0 where the fabric offers no multicast
        arr = (ctypes.c_void_p * self.world)(*ptrs)
        _l.call("gb_comm_attach", _l.I(self.rank), _l.I(self.world), arr, ctypes.c_void_p(mc))
        self._symm_handle, self._symm_tensor = hdl, t
        self._raw.append(t)
        self._ipc = True
        self.multicast = mc != 0
        dist.barrier(group=process_group)
        return True

    def view(self, offset_bytes: int, numel: int, dtype: torch.dtype, rank: int = 0) -> torch.Tensor:
        """A typed view of ``numel`` elements at ``offset_bytes`` of the data region
        (``rank`` selects the emulated rank's buffer; real runs only see their own)."""
        esz = torch.empty((), dtype=dtype).element_size()
        raw = self._raw[rank if self.emulate else 0]
        lo = self.flag_bytes + offset_bytes
        return raw[lo:lo + numel * esz].view(dtype)

    def abs_offset(self, offset_bytes: int) -> int:
        return self.flag_bytes + offset_bytes

    # ---- collectives ------------------------------------------------------------------
    OPT_KINDS = {"adamw": 0, "sgd": 1, "lion": 2}

    def fused_step(self, mode: int, dtype: torch.dtype, grad_off: int, param_off: int, n: int,
                   master, m, v, hyper, ctas: int = 32, hyper_dev: torch.Tensor = None, kind: str = "adamw",
                   phase: int = 0, wd_mask=None, gshard=None, sqpart=None):
        """See ``gb_comm_fused_step2``.  master/m/v: tensors (lists of tensors when emulating).
        ``hyper_dev``: a device tensor of the same eight floats, read by the kernel when it
        runs (for launches captured in a CUDA graph, and for the clip factor).  ``kind``: the
        optimizer; ``phase``: 0 whole step, 1 reduce-scatter into ``gshard`` with sums of squares
        in ``sqpart``, 2 update from ``gshard`` and all-gather; ``wd_mask``: uint8 per 8 shard
        elements, 0 = no weight decay."""
        if self.host:
            return self._fused_step_host(mode, dtype, grad_off, param_off, n, master, m, v, hyper, kind, phase,
                                         wd_mask, gshard, sqpart)

        def arr(x):
            if x is None:
                return None
            xs = x if isinstance(x, (list, tuple)) else [x]
            return (ctypes.c_void_p * len(xs))(*[t.data_ptr() for t in xs])
        hy = (ctypes.c_float * 8)(*[float(h) for h in hyper])
        code = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}[dtype]
        _l.call("gb_comm_fused_step2", _l.I(mode), _l.I(code),
                _l.L(self.abs_offset(grad_off)), _l.L(self.abs_offset(param_off)), _l.L(n),
                arr(master), arr(m), arr(v), hy, _l.ptr(hyper_dev), _l.I(self.OPT_KINDS[kind]), _l.I(phase),
                arr(wd_mask), arr(gshard), arr(sqpart), _l.I(ctas), _l.I(1 if self.emulate else 0),
                _l.stream_ptr())

    def all_reduce(self, offset_bytes: int, n: int, dtype: torch.dtype, op: str = "sum", ctas: int = 64):
        """In-place all-reduce (``sum`` or ``mean``) of ``n`` elements at ``offset_bytes`` of
        every rank's symmetric buffer: two-shot (each rank reduces one slice in rank order
        through peer loads and writes it back to every peer).  ``n`` must be a multiple of
        ``world * 8``; fp16 / bf16 / fp32."""
        scale = float(self.world) if op == "sum" else 1.0
        esz = torch.empty((), dtype=dtype).element_size()
        slot = self.ONESHOT_BYTES // (2 * self.world) // 16 * 16
        if not self.host and self.world > 1 and n * esz <= min(slot, 256 << 10) and (n * esz) % 16 == 0:
            # short vectors: push + one barrier + local sum (two barriers and a round trip less)
            code = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}[dtype]
            nb = n * esz
            ctas1 = 1 if nb <= (8 << 10) else min(ctas, max(1, nb // (8 << 10)))
            _l.call("gb_comm_allreduce_oneshot", _l.I(code), _l.L(self.abs_offset(offset_bytes)), _l.L(n),
                    _l.L(self.abs_offset(self.user_bytes)), _l.L(slot), _l.F(scale / self.world), _l.I(ctas1),
                    _l.I(1 if self.emulate else 0), _l.stream_ptr())
            return
        self.fused_step(0, dtype, offset_bytes, offset_bytes, n, None, None, None,
                        [0, 0, 0, 0, 0, 1, 1, scale], ctas)

    def _fused_step_host(self, mode, dtype, grad_off, param_off, n, master, m, v, hyper, kind="adamw", phase=0,
                         wd_mask=None, gshard=None, sqpart=None):
        """Restatement of the kernel's arithmetic on the host (fp32, same operation order):
        mean of the gradients over ranks, then either the mean written back (mode 0) or the
        optimizer on the slice this rank owns followed by an all-gather of the updated parameters."""
        lr, wd, b1, b2, eps, bc1, bc2, gscale = [float(h) for h in hyper]
        W = self.world
        L = n // W
        if phase == 2:
            g = gshard * gscale
        else:
            g = self.view(grad_off, n, dtype).float()
            if W > 1:
                import torch.distributed as dist
                dist.all_reduce(g, group=self._pg)
                g /= W
            if phase == 1:
                gshard.copy_(g[self.rank * L:(self.rank + 1) * L])
                sqpart.zero_()
                sqpart[0] = (gshard * gshard).sum()
                return
            g = g * gscale
            if mode == 0:
                self.view(grad_off, n, dtype).copy_(g.to(dtype))
                return
            g = g[self.rank * L:(self.rank + 1) * L]
        p = master
        wdv = wd if wd_mask is None else wd * wd_mask.to(torch.float32).repeat_interleave(8)
        if kind == "adamw":
            p.mul_(1 - lr * wdv)
            m.mul_(b1).add_(g, alpha=1 - b1)
            v.mul_(b2).addcmul_(g, g, value=1 - b2)
            p.sub_(lr * (m / bc1) / ((v / bc2).sqrt() + eps))
        elif kind == "sgd":
            m.mul_(b1).add_(g + wdv * p)
            p.sub_(lr * m)
        else:
            c = b1 * m + (1 - b1) * g
            p.sub_(lr * (torch.sign(c) + wdv * p))
            m.mul_(b2).add_(g, alpha=1 - b2)
        out = self.view(param_off, n, dtype)
        if W == 1:
            out.copy_(p.to(dtype))
            return
        import torch.distributed as dist
        mine = p.to(dtype).contiguous().view(torch.uint8)
        parts = [torch.empty_like(mine) for _ in range(W)]
        dist.all_gather(parts, mine, group=self._pg)
        out.view(torch.uint8).copy_(torch.cat(parts))

    def allreduce_small(self, vec, slot_off: int):
        """In-place sum over ranks of a short fp32 vector (list of vectors when emulating)."""
        if self.host:
            if self.world > 1:
                import torch.distributed as dist
                dist.all_reduce(vec, group=self._pg)
            return
        xs = vec if isinstance(vec, (list, tuple)) else [vec]
        n = xs[0].numel()
        if n * self.world * 4 > (1 << 20):
            raise ValueError("allreduce_small: vector too long for the exchange area")
        arr = (ctypes.c_void_p * len(xs))(*[t.data_ptr() for t in xs])
        _l.call("gb_comm_allreduce_small", arr, _l.I(n), _l.L(self.abs_offset(slot_off)),
                _l.I(1 if self.emulate else 0), _l.stream_ptr())

    def broadcast(self, root: int, offset_bytes: int, nbytes: int, ctas: int = 16):
        if self.host:
            if self.world > 1:
                import torch.distributed as dist
                dist.broadcast(self._raw[0][offset_bytes:offset_bytes + nbytes], src=root, group=self._pg)
            return
        _l.call("gb_comm_broadcast", _l.I(root), _l.L(self.abs_offset(offset_bytes)), _l.L(nbytes),
                _l.I(ctas), _l.I(1 if self.emulate else 0), _l.stream_ptr())

    def barrier(self):
        if self.host:
            if self.world > 1:
                import torch.distributed as dist
                dist.barrier(group=self._pg)
            return
        _l.call("gb_comm_barrier", _l.I(1 if self.emulate else 0), _l.stream_ptr())

    def check(self):
        """Raises ``CollectiveTimeout`` if a kernel gave up waiting (synchronises)."""
        if self.host:
            return
        code, detail, block, count = _l.read_status()
        if code == 3:
            raise CollectiveTimeout(f"collective wait ran out of budget (detail {detail}, block {block})")
        if code != 0:
            raise _l.KernelStatusError(f"kernel status {code} (detail {detail}, block {block})")

    def close(self):
        if getattr(self, "_ipc", False):
            torch.cuda.synchronize()
            if self._symm_handle is not None and self.world > 1:
                # every rank stops using the multicast mapping before any rank releases it
                import torch.distributed as dist
                dist.barrier(group=self._pg)
            self._raw.clear()
            _l.call("gb_comm_free")
            self._symm_handle = self._symm_tensor = None
            self._ipc = False

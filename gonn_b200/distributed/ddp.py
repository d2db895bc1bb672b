"""Data-parallel engine over symmetric peer memory.

``DistributedDataParallel`` re-homes a module's parameters and gradients in two
flat regions of this rank's symmetric buffer, cuts them into buckets, and hands
each bucket to ONE kernel as soon as backward has produced its gradients:

* ``optimizer=None``: the kernel leaves the mean gradient on every rank
  (all-reduce-mean); any optimizer can then step (``DDPStep`` semantics of the
  reference, distributed/distributed.go:422-428).
* ``optimizer={"kind": "adamw" | "sgd" | "lion", ...}``: the kernel reduce-scatters the
  bucket, runs the optimizer on the shard this rank owns (fp32 master and moments: 1/W of
  the state per rank, ZeRO-1) and all-gathers the updated 16-bit parameters — gradient
  collective, scale/cast, optimizer and parameter collective in one launch, overlapped
  with the rest of backward on a side stream.  Options: ``lr``, ``weight_decay``, ``betas``
  (AdamW, Lion), ``momentum`` (SGD), ``eps``; ``no_decay`` (a predicate on ``(name,
  parameter)`` or ``"1d"`` for every vector-shaped parameter: biases and norm weights) exempts
  parameters from weight decay; ``max_grad_norm`` clips by the global norm as the reference's
  ``ClipGradNorm`` does (optim/clip.go:23-65): the reduce-scatter then still overlaps with
  backward (it leaves the averaged shard in fp32 and its sum of squares), and the updates
  run once the norm of all buckets is known.

The reference reduces one flat vector after the whole backward, through rank 0
over TCP, without overlap or bucketing (distributed.go:249-293, :84-86).  Kept
from it: the mean over ranks, a gradient that is missing on a rank counts as
zeros, and every rank ends a step with bit-identical parameters.

Layers cooperate through *gradient sinks*: an op that computes a parameter
gradient writes it straight into the bucket (``param._gb_sink``) and reports the
parameter ready; gradients that arrive through autograd's own accumulation are
caught by a post-accumulate hook.
"""
from __future__ import annotations

import contextlib
from typing import Dict, List, Optional

import torch

from .nvlink import SymmetricMemory

_SLOT_BYTES = 1 << 20


def ordered_parameters(module: torch.nn.Module) -> List[torch.nn.Parameter]:
    """Trainable parameters in registration order, except that groups a module declares in
    ``fuse_groups()`` are kept adjacent (e.g. the q/k/v weights of an attention layer)."""
    fused: Dict[int, List[torch.nn.Parameter]] = {}
    for m in module.modules():
        fg = getattr(m, "fuse_groups", None)
        if fg is None:
            continue
        for grp in fg():
            grp = [p for p in grp if p is not None and p.requires_grad]
            for p in grp:
                fused[id(p)] = grp
    out, seen = [], set()
    for p in module.parameters():
        if not p.requires_grad or id(p) in seen:
            continue
        for q in fused.get(id(p), [p]):
            if id(q) not in seen:
                seen.add(id(q))
                out.append(q)
    return out


def plan_buckets(sizes, world: int, limit: int):
    """Layout of the flat parameter / gradient buffers.

    Parameters are packed in order, each starting on an 8-element boundary (16 bytes for 16-bit
    types: the alignment the vector and TMA accesses need).  A bucket is closed once it holds at
    least ``limit`` elements and is padded to a multiple of ``world * 8`` elements, so that it
    splits into ``world`` shards of whole 16-byte vectors.  Returns ``(offsets, buckets, total)``:
    the offset of every parameter, ``(start, length, member indices)`` per bucket, and the
    buffer length in elements."""
    align = world * 8
    limit = max(int(limit), align)
    offsets, buckets = [], []
    off = start = 0
    members = []
    for i, n in enumerate(sizes):
        offsets.append(off)
        members.append(i)
        off += (int(n) + 7) // 8 * 8
        if off - start >= limit:
            off = start + (off - start + align - 1) // align * align
            buckets.append((start, off - start, members))
            start, members = off, []
    if members:
        off = start + (off - start + align - 1) // align * align
        buckets.append((start, off - start, members))
    return offsets, buckets, off


class _Bucket:
    __slots__ = ("index", "start", "length", "params", "pending", "launched", "master", "m", "v", "wd_mask", "gshard")

    def __init__(self, index, start):
        self.index, self.start, self.length = index, start, 0
        self.params: List[torch.nn.Parameter] = []
        self.pending = 0
        self.launched = False
        self.master = self.m = self.v = self.wd_mask = self.gshard = None


class DistributedDataParallel(torch.nn.Module):
    def __init__(self, module: torch.nn.Module, process_group=None, optimizer: Optional[dict] = None,
                 bucket_mb: float = 32.0, comm_ctas: Optional[int] = None, overlap: bool = True,
                 rank: Optional[int] = None, world: Optional[int] = None):
        super().__init__()
        self.module = module
        if rank is None or world is None:
            import torch.distributed as dist
            if dist.is_available() and dist.is_initialized():
                rank, world = dist.get_rank(process_group), dist.get_world_size(process_group)
            else:
                rank, world = 0, 1
        self.rank, self.world = rank, world
        # one rank: the step kernel is a plain memory-bound pass and may fill the GPU; several
        # ranks: it runs beside backward, so it gets a slice of the SMs
        self.overlap = overlap
        self.comm_ctas = comm_ctas if comm_ctas is not None else (296 if world == 1 else 48)
        params = ordered_parameters(module)
        if not params:
            raise ValueError("DistributedDataParallel: the module has no trainable parameters")
        dt = params[0].dtype
        dev = params[0].device
        if dt == torch.float32:
            if optimizer is not None:
                raise TypeError("DistributedDataParallel: the fused sharded optimizer needs bf16/fp16 "
                                "parameters; fp32 parameters are all-reduced (optimizer=None)")
        elif dt not in (torch.bfloat16, torch.float16):
            raise TypeError("DistributedDataParallel: parameters must be bf16/fp16/fp32; use "
                            "distributed.Group (TCP) for fp64 data parallelism")
        self._esz = 4 if dt == torch.float32 else 2
        self.host = dev.type != "cuda"
        if self.host and world != 1:
            # CPU ranks: the same engine (buckets, hooks, sharded state) with the collectives
            # carried by torch.distributed's CPU backend instead of the peer-memory kernels
            import torch.distributed as dist
            if not (dist.is_available() and dist.is_initialized()):
                raise TypeError("DistributedDataParallel: multi-rank runs on the host need an "
                                "initialised torch.distributed process group (gloo)")
        if any(p.dtype != dt or p.device != dev for p in params):
            raise TypeError("DistributedDataParallel: all parameters must share dtype and device")
        self.dtype, self.device = dt, dev
        self.params = params

        # ---- layout -------------------------------------------------------------------
        limit = int(bucket_mb * (1 << 20) / self._esz)
        offsets, spans, self.total = plan_buckets([p.numel() for p in params], world, limit)
        self.buckets: List[_Bucket] = []
        self._where: Dict[int, tuple] = {}
        for start, length, members in spans:
            b = _Bucket(len(self.buckets), start)
            b.length = length
            for i in members:
                b.params.append(params[i])
                self._where[id(params[i])] = (b, offsets[i], params[i].numel())
            self.buckets.append(b)
        nbytes = self.total * self._esz
        self._param_off = _SLOT_BYTES
        self._grad_off = _SLOT_BYTES + (nbytes + 255) // 256 * 256
        self.symm = SymmetricMemory(self._grad_off + nbytes, rank, world, process_group, device=dev)
        self.flat_params = self.symm.view(self._param_off, self.total, dt)
        self.flat_grads = self.symm.view(self._grad_off, self.total, dt)

        # ---- re-home parameters and gradients ---------------------------------------------
        with torch.no_grad():
            for p in params:
                _, o, n = self._where[id(p)]
                dst = self.flat_params[o:o + n].view(p.shape)
                dst.copy_(p.data)
                p.data = dst
                p.grad = self.flat_grads[o:o + n].view(p.shape)
                p._gb_sink = self
                p.register_post_accumulate_grad_hook(self._autograd_hook)
        if world > 1:
            # every rank starts from rank 0's values (BroadcastParams of the reference)
            self.symm.broadcast(0, self._param_off, self.total * self._esz)
            if not self.host:
                torch.cuda.synchronize()

        self._fresh = {id(p): True for p in params}
        self._autograd_params: Dict[int, torch.nn.Parameter] = {}
        self._sync = True
        self._comm_stream = None if self.host else torch.cuda.Stream(device=dev, priority=-1)
        self.t = 0
        self.opt = dict(optimizer) if optimizer is not None else None
        self._hyper_dev = None      # device copy of the optimizer scalars (captured launches, clip factor)
        self._capturing = False     # True while a step is being captured into a CUDA graph
        self.kind = "adamw"
        self.max_grad_norm = None
        self.grad_norm = None       # device scalar: the global gradient norm of the last clipped step
        if self.opt is not None:
            kind = self.opt.get("kind", "adamw").lower()
            if kind not in ("adamw", "sgd", "lion"):
                raise ValueError("DistributedDataParallel: the fused sharded optimizer is one of adamw, sgd, lion")
            self.kind = kind
            self.lr = float(self.opt.get("lr", 1e-3))
            self.weight_decay = float(self.opt.get("weight_decay", 0.01 if kind == "adamw" else 0.0))
            default_betas = (0.9, 0.99) if kind == "lion" else (0.9, 0.999)
            self.betas = tuple(self.opt.get("betas", default_betas))
            if kind == "sgd":
                self.betas = (float(self.opt.get("momentum", 0.9)), 0.0)
            self.eps = float(self.opt.get("eps", 1e-8))
            mg = self.opt.get("max_grad_norm")
            self.max_grad_norm = float(mg) if mg is not None else None
            # which parameters are exempt from weight decay: one byte per 8 elements of the flat layout
            no_decay = self.opt.get("no_decay")
            mask_full = None
            if no_decay is not None:
                names = {id(p): n for n, p in module.named_parameters()}
                mask_full = torch.ones(self.total // 8, dtype=torch.uint8)
                for p in params:
                    exempt = (p.dim() <= 1) if no_decay == "1d" else bool(no_decay(names.get(id(p), ""), p))
                    if exempt:
                        _, o, n = self._where[id(p)]
                        mask_full[o // 8:(o + n + 7) // 8] = 0
                mask_full = mask_full.to(dev)
            for b in self.buckets:
                L = b.length // world
                lo = b.start + rank * L
                b.master = self.flat_params[lo:lo + L].to(torch.float32)
                b.m = torch.zeros(L, dtype=torch.float32, device=dev)
                b.v = torch.zeros(L, dtype=torch.float32, device=dev) if kind == "adamw" else None
                b.wd_mask = mask_full[lo // 8:(lo + L) // 8].contiguous() if mask_full is not None else None
                if self.max_grad_norm is not None:
                    b.gshard = torch.zeros(L, dtype=torch.float32, device=dev)
            if self.max_grad_norm is not None:
                nb = len(self.buckets)
                self._sq = torch.zeros(nb * self.comm_ctas, dtype=torch.float32, device=dev)
                self._sq_total = torch.zeros(max(world, 1), dtype=torch.float32, device=dev)
                self.grad_norm = torch.zeros(1, dtype=torch.float32, device=dev)
                self._hyper_dev = torch.zeros(8, dtype=torch.float32, device=dev)
        self._reset_step()

    # ---- CUDA-graph support (gonn_b200.utils.graph.GraphedStep) -----------------------------------
    def graph_hyper_buffer(self) -> torch.Tensor:
        """Device copy of the eight optimizer scalars that captured launches read at run time."""
        if self._hyper_dev is None:
            self._hyper_dev = torch.zeros(8, dtype=torch.float32, device=self.device)
        return self._hyper_dev

    # ---- sink protocol (called by ops) ------------------------------------------------------
    def target(self, p):
        """(flat gradient view of ``p``, whether it has not been written yet this step)."""
        _, o, n = self._where[id(p)]
        return self.flat_grads[o:o + n], self._fresh[id(p)]

    def ready(self, p):
        self._fresh[id(p)] = False
        self._mark(p)

    def _autograd_hook(self, p):
        # The hook also fires when the producing op returned no gradient because it had
        # already written into the bucket through the sink: nothing to do then.
        if id(p) in self._ready:
            return
        # autograd added into p.grad (our flat view); make sure that is still the case
        _, o, n = self._where[id(p)]
        view = self.flat_grads[o:o + n].view(p.shape)
        if p.grad is None or p.grad.data_ptr() != view.data_ptr():
            if p.grad is not None:
                if self._fresh[id(p)]:
                    view.copy_(p.grad)
                else:
                    view.add_(p.grad)
            p.grad = view
        self._autograd_params[id(p)] = p
        self._fresh[id(p)] = False
        self._mark(p)

    def _mark(self, p):
        b = self._where[id(p)][0]
        if id(p) in self._ready:
            # a second contribution in one backward (a shared parameter): it was accumulated
            # into the bucket, but if the bucket has already been reduced it is too late
            if b.launched and self._sync and self.overlap:
                raise RuntimeError("a gradient arrived after its bucket was reduced (a parameter is "
                                   "used more than once); construct the wrapper with overlap=False")
            return
        self._ready.add(id(p))
        b.pending -= 1
        if b.pending == 0 and self._sync and self.overlap:
            self._launch_ready()

    def _launch_ready(self):
        """Launches buckets strictly in descending index: a complete bucket waits until every
        bucket above it has been launched.  Collectives of different ranks are matched by
        launch order alone, and which gradients arrive first (or at all) may differ from rank
        to rank, so the order must not depend on it; ``step`` flushes the rest the same way."""
        while self._next >= 0 and self.buckets[self._next].pending == 0:
            b = self.buckets[self._next]
            self._next -= 1
            self._launch(b)

    # ---- bucket launch ------------------------------------------------------------------------
    def _hyper(self):
        if self.opt is None:
            return [0, 0, 0, 0, 0, 1, 1, 1.0]
        t = self.t + 1
        b1, b2 = self.betas
        if self.kind != "adamw":
            return [self.lr, self.weight_decay, b1, b2, self.eps, 1.0, 1.0, 1.0]
        return [self.lr, self.weight_decay, b1, b2, self.eps, 1 - b1 ** t, 1 - b2 ** t, 1.0]

    def _launch(self, b: _Bucket):
        b.launched = True
        if self.world == 1 and self.opt is None:
            return  # nothing to reduce and nobody to update
        clip = self.opt is not None and self.max_grad_norm is not None
        args = (1 if self.opt is not None else 0, self.dtype, self._grad_off + b.start * self._esz,
                self._param_off + b.start * self._esz, b.length, b.master, b.m, b.v, self._hyper(), self.comm_ctas,
                self._hyper_dev if (self._capturing or clip) else None)
        kw = dict(kind=self.kind, wd_mask=b.wd_mask)
        if clip:
            # phase 1 now (overlapped with backward): reduce-scatter, fp32 shard and its sum of squares;
            # the update waits in step() for the norm of all buckets
            kw.update(phase=1, gshard=b.gshard,
                      sqpart=self._sq[b.index * self.comm_ctas:(b.index + 1) * self.comm_ctas])
        if self.host:
            self.symm.fused_step(*args, **kw)
            return
        cur = torch.cuda.current_stream()
        self._comm_stream.wait_stream(cur)
        with torch.cuda.stream(self._comm_stream):
            self.symm.fused_step(*args, **kw)
        self._launched_any = True

    def _clip_and_update(self):
        """Second half of a clipped step: global norm from the per-bucket sums of squares (summed
        over ranks: every rank holds a disjoint shard), clip factor on the device, then the
        optimizer update and parameter all-gather of every bucket."""
        from .. import lib as _l
        import ctypes
        hy = self._hyper()
        if self.host:
            total = self._sq.sum().reshape(1)
            if self.world > 1:
                import torch.distributed as dist
                dist.all_reduce(total)
            norm = float(total.sqrt())
            scale = min(1.0, self.max_grad_norm / (norm + 1e-6))
            self.grad_norm.fill_(norm)
            hy[7] = scale
            for b in reversed(self.buckets):
                self.symm.fused_step(1, self.dtype, self._grad_off + b.start * self._esz,
                                     self._param_off + b.start * self._esz, b.length, b.master, b.m, b.v, hy,
                                     self.comm_ctas, None, kind=self.kind, phase=2, wd_mask=b.wd_mask, gshard=b.gshard)
            return
        ctx = torch.cuda.stream(self._comm_stream)
        with ctx:
            if not self._capturing:
                # the scalars of this step; element 7 is overwritten by the clip kernel below
                _l.call("gb_set_words", None, ctypes.c_uint(0), ctypes.c_uint(0), _l.ptr(self._hyper_dev),
                        (ctypes.c_float * 8)(*[float(h) for h in hy]), _l.stream_ptr())
            _l.call("gb_comm_sum_partials", _l.ptr(self._sq), _l.I(self._sq.numel()), _l.ptr(self._sq_total),
                    _l.stream_ptr())
            if self.world > 1:
                self.symm.allreduce_small(self._sq_total[:1], 0)
            _l.call("gb_comm_clip_scale", _l.ptr(self._sq_total), _l.I(1), _l.F(self.max_grad_norm),
                    _l.ptr(self._hyper_dev), _l.ptr(self.grad_norm), _l.stream_ptr())
            for b in reversed(self.buckets):
                self.symm.fused_step(1, self.dtype, self._grad_off + b.start * self._esz,
                                     self._param_off + b.start * self._esz, b.length, b.master, b.m, b.v, hy,
                                     self.comm_ctas, self._hyper_dev, kind=self.kind, phase=2, wd_mask=b.wd_mask,
                                     gshard=b.gshard)

    def _reset_step(self):
        self._ready = set()
        self._launched_any = False
        self._next = len(self.buckets) - 1      # next bucket to launch (descending order)
        for b in self.buckets:
            b.pending = len(b.params)
            b.launched = False

    # ---- user interface -------------------------------------------------------------------------
    def forward(self, *a, **kw):
        return self.module(*a, **kw)

    @contextlib.contextmanager
    def no_sync(self):
        """Accumulate gradients locally: no collective, no update, until the next
        backward outside this context."""
        old = self._sync
        self._sync = False
        try:
            yield
        finally:
            self._sync = old
            # parameters stay "written" so that the next backward accumulates
            self._ready = set()
            for b in self.buckets:
                b.pending = len(b.params)

    def step(self):
        """Finishes the step: reduces buckets that are still pending, waits for the side
        stream, and prepares the gradient buffers for the next backward."""
        for p in self.params:
            if self._fresh[id(p)]:
                # no gradient this step on this rank: contributes zeros, like a nil grad
                # in the reference (distributed.go:253-258)
                _, o, n = self._where[id(p)]
                self.flat_grads[o:o + n].zero_()
        while self._next >= 0:                 # the rest, in the same descending order
            b = self.buckets[self._next]
            self._next -= 1
            self._launch(b)
        if self.opt is not None and self.max_grad_norm is not None:
            self._clip_and_update()
        if self._launched_any:
            torch.cuda.current_stream().wait_stream(self._comm_stream)
        self.t += 1
        for k in self._fresh:
            self._fresh[k] = True
        if self.opt is not None:
            # the fused optimizer has consumed the gradients; those that autograd accumulates
            # in place must start the next step from zero
            for p in self._autograd_params.values():
                _, o, n = self._where[id(p)]
                self.flat_grads[o:o + n].zero_()
        # all-reduce mode: the averaged gradients stay readable in ``p.grad`` for the caller's
        # optimizer, which clears them (``zero_grad``) before the next backward as usual
        self._reset_step()

    synchronize = step

    def zero_grad(self):
        self.flat_grads.zero_()
        for k in self._fresh:
            self._fresh[k] = True

    def check(self):
        self.symm.check()

    def state_bytes_per_rank(self) -> int:
        if self.opt is None:
            return 0
        per = (3 if self.kind == "adamw" else 2) * 4        # master + moments, fp32
        return sum(per * (b.length // self.world) for b in self.buckets)

    def close(self):
        self.symm.close()

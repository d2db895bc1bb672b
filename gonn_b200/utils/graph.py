"""A whole training step as one CUDA graph.

``GraphedStep(step_fn, ddp, example_inputs)`` runs ``step_fn(*inputs)`` (forward, backward and
``ddp.step()``; it returns the loss) a few times eagerly, captures one more run into a CUDA
graph and from then on replays it: one graph launch per step instead of several hundred kernel
launches issued from Python.  The reference has no counterpart (its training loop is a host
loop over tape nodes, nn/module.go and optim/*.go); this is the launch-bound inner loop captured
as the CUDA execution model suggests.

What changes from step to step is kept out of the captured kernel arguments:

* inputs are copied into static device buffers before each replay;
* the optimizer scalars (learning rate, Adam bias corrections) are read by the fused
  data-parallel step from a small device buffer that is rewritten before each replay;
* barrier epochs and flag serial numbers of the peer-memory collectives are captured relative
  to two device words; fresh bases are reserved and written before each replay, so flags are
  never reused (``gb_comm_capture_begin`` / ``gb_comm_reserve`` in csrc/comm.cu).

Limits: the step must be static (same shapes, same control flow), must not synchronise with
the host, and layers that draw random numbers per call (dropout with p > 0 in training mode)
would replay the same mask; ``GraphedStep`` refuses modules with active dropout.
"""
from __future__ import annotations

import ctypes
from typing import Callable, Sequence

import torch

from .. import lib as _l


def _active_dropout(module: torch.nn.Module) -> bool:
    for m in module.modules():
        p = getattr(m, "p", None)
        if "Dropout" in type(m).__name__ and isinstance(p, (int, float)) and p > 0 and m.training:
            return True
    return False


class GraphedStep:
    def __init__(self, step_fn: Callable[..., torch.Tensor], ddp, example_inputs: Sequence[torch.Tensor],
                 warmup: int = 3):
        if not example_inputs or not all(t.is_cuda for t in example_inputs):
            raise ValueError("GraphedStep: example inputs must be CUDA tensors")
        if _active_dropout(ddp.module):
            raise ValueError("GraphedStep: a captured step would replay the same dropout mask; "
                             "set p = 0 or call eval() on the dropout layers")
        self.ddp = ddp
        self.step_fn = step_fn
        self.inputs = [t.clone() for t in example_inputs]
        dev = self.inputs[0].device
        self._bases = torch.zeros(2, dtype=torch.int32, device=dev)       # epoch base, serial base
        self._counts = (ctypes.c_uint * 2)()
        self._launches_per_step = 0
        ddp.graph_hyper_buffer()
        # eager runs on a side stream first: lazy initialisation (kernel attributes, index maps,
        # scratch buffers, autograd state) must not happen inside the capture
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(warmup):
                step_fn(*self.inputs)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        t_before = ddp.t
        k0 = _l.kernel_count
        _l.call("gb_comm_capture_begin", _l.ptr(self._bases))
        ddp._capturing = True
        try:
            with torch.cuda.graph(self.graph):
                self.loss = step_fn(*self.inputs)
        finally:
            ddp._capturing = False
            _l.lib().gb_comm_capture_end(self._counts)
        self._launches_per_step = _l.kernel_count - k0
        ddp.t = t_before                     # the capture ran no kernel: it was not a step

    def __call__(self, *inputs: torch.Tensor) -> torch.Tensor:
        """Copies ``inputs`` into the static buffers (skipped for a tensor that already is the
        static buffer), replays the step and returns the static loss tensor."""
        for dst, src in zip(self.inputs, inputs):
            if src is not dst:
                dst.copy_(src, non_blocking=True)
        out = (ctypes.c_uint * 2)()
        _l.lib().gb_comm_reserve(ctypes.c_uint(self._counts[0]), ctypes.c_uint(self._counts[1]), out)
        hy = (ctypes.c_float * 8)(*[float(h) for h in self.ddp._hyper()])
        # one small launch carries the values as kernel arguments (stream-ordered, no host
        # buffer whose lifetime would matter)
        _l.call("gb_set_words", _l.ptr(self._bases), ctypes.c_uint(out[0]), ctypes.c_uint(out[1]),
                _l.ptr(self.ddp.graph_hyper_buffer()), hy, _l.stream_ptr())
        self.graph.replay()
        self.ddp.t += 1
        _l.kernel_count += self._launches_per_step
        return self.loss

    @property
    def launches_per_step(self) -> int:
        """Kernels of this library inside one replay (counted while capturing)."""
        return self._launches_per_step

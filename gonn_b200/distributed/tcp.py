"""CPU process group over TCP, wire-compatible with the reference's star protocol.

Frame: ``[1 B op][8 B big-endian count][count x 8 B big-endian IEEE-754 float64]``;
op codes 1 = AllReduce(mean), 2 = Broadcast, 3 = Barrier, 4 = AllReduceSum; the
handshake is 8 bytes (magic 0x60DDDD90, rank) answered by an empty Barrier frame
(distributed/distributed.go:18-24, 109-117, 146-227, 471-506).  Rank 0 is the
coordinator: it gathers in rank order 1..W-1, reduces, and sends the same bytes to
everyone, so all ranks end with bit-identical values.

Beyond the reference: every socket operation has a deadline (``timeout``) and
failures surface as typed exceptions (``PeerTimeout``, ``ProtocolError``,
``PeerClosed``) instead of blocking forever; a collective on a closed group raises
``GroupClosed``.
"""
from __future__ import annotations

import socket
import struct
import time
from typing import List, Optional, Sequence

import numpy as np
import torch

OP_ALLREDUCE, OP_BROADCAST, OP_BARRIER, OP_ALLREDUCE_SUM = 1, 2, 3, 4
MAGIC = 0x60DDDD90
DialTimeout = 15.0  # seconds a non-zero rank keeps dialling the coordinator


class DistributedError(RuntimeError):
    pass


class PeerTimeout(DistributedError):
    """A peer did not answer within the deadline."""


class PeerClosed(DistributedError):
    """A peer closed its connection in the middle of a collective."""


class ProtocolError(DistributedError):
    """A frame carried the wrong op code or element count (ranks diverged)."""


class GroupClosed(DistributedError):
    pass


def _recv_into(c: socket.socket, view: memoryview, who: str) -> None:
    """Fills ``view`` (bytes) from the socket: no intermediate copies."""
    got, n = 0, len(view)
    while got < n:
        try:
            k = c.recv_into(view[got:], min(n - got, 1 << 22))
        except socket.timeout:
            raise PeerTimeout(f"timed out waiting for {who}") from None
        except OSError as e:
            raise PeerClosed(f"connection to {who} failed: {e}") from None
        if k == 0:
            raise PeerClosed(f"{who} closed the connection")
        got += k


def _recv_exact(c: socket.socket, n: int, who: str) -> bytes:
    buf = bytearray(n)
    _recv_into(c, memoryview(buf), who)
    return bytes(buf)


def write_frame(c: socket.socket, op: int, vals: Optional[np.ndarray], who: str = "peer",
                scratch: Optional[np.ndarray] = None, prepared: bool = False) -> None:
    """Writes one frame; ``scratch`` (a ``>f8`` array of the same size) holds the byte-swapped payload
    (already filled by the caller when ``prepared``)."""
    n = 0 if vals is None else int(vals.size)
    try:
        if n == 0:
            c.sendall(struct.pack(">BQ", op, 0))
        elif n <= 1024:
            c.sendall(struct.pack(">BQ", op, n) + np.ascontiguousarray(vals, dtype=">f8").tobytes())
        else:
            # one byte-swapping pass, then the socket reads the array's memory directly
            if scratch is not None and scratch.size == n:
                be = scratch
                if not prepared:
                    be[...] = vals.reshape(-1)
            else:
                be = np.ascontiguousarray(vals, dtype=">f8")
            c.sendall(struct.pack(">BQ", op, n))
            c.sendall(memoryview(be).cast("B"))
    except socket.timeout:
        raise PeerTimeout(f"timed out sending to {who}") from None
    except OSError as e:
        raise PeerClosed(f"connection to {who} failed: {e}") from None


def read_frame(c: socket.socket, want_op: int, want_n: int, who: str = "peer",
               into: Optional[np.ndarray] = None) -> np.ndarray:
    """Reads one frame; ``into`` (a ``>f8`` array of ``want_n`` elements) receives the payload in place."""
    op, n = struct.unpack(">BQ", _recv_exact(c, 9, who))
    if op != want_op:
        raise ProtocolError(f"{who}: expected op {want_op}, got {op} (ranks called different collectives)")
    if n != want_n:
        raise ProtocolError(f"{who}: expected {want_n} elements, got {n}")
    if n == 0:
        return np.empty(0, dtype=np.float64)
    arr = np.empty(n, dtype=">f8") if into is None else into
    _recv_into(c, memoryview(arr).cast("B"), who)
    if arr.dtype.byteorder == ">":                      # a little-endian host: swap in place, reinterpret
        return arr.byteswap(inplace=True).view(np.float64)
    return arr.view(np.float64)


def _tune(c: socket.socket) -> None:
    """No Nagle delay, and socket buffers large enough for a gradient frame to move in few wake-ups."""
    c.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
    for opt in (socket.SO_SNDBUF, socket.SO_RCVBUF):
        try:
            c.setsockopt(socket.SOL_SOCKET, opt, 4 << 20)
        except OSError:
            pass


class Group:
    """A connected group of ``world`` CPU ranks; rank 0 listens on ``peers[0]``."""

    def __init__(self, rank: int, world: int, peers: Sequence[str], timeout: float = 30.0):
        if world < 1 or not (0 <= rank < world):
            raise ValueError(f"distributed.Init: bad rank/world {rank}/{world}")
        self.rank, self.world, self.timeout = rank, world, timeout
        self.conns: List[Optional[socket.socket]] = []
        self.lis: Optional[socket.socket] = None
        self.closed = False
        if world == 1:
            return
        host, port = peers[0].rsplit(":", 1)
        if rank == 0:
            lis = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
            lis.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
            lis.bind((host, int(port)))
            lis.listen(world)
            lis.settimeout(max(timeout, DialTimeout))
            self.lis = lis
            self.conns = [None] * world
            try:
                for _ in range(1, world):
                    try:
                        c, addr = lis.accept()
                    except socket.timeout:
                        raise PeerTimeout("distributed.Init: a rank never connected") from None
                    c.settimeout(timeout)
                    _tune(c)
                    magic, r = struct.unpack(">II", _recv_exact(c, 8, f"client {addr}"))
                    if magic != MAGIC:
                        raise ProtocolError(f"distributed.Init: bad handshake magic from {addr}")
                    if r < 1 or r >= world or self.conns[r] is not None:
                        raise ProtocolError(f"distributed.Init: invalid or duplicate rank {r} in handshake")
                    self.conns[r] = c
                for r in range(1, world):
                    write_frame(self.conns[r], OP_BARRIER, None, f"rank {r}")
            except Exception:
                self.Close()
                raise
        else:
            deadline = time.time() + DialTimeout
            while True:
                try:
                    c = socket.create_connection((host, int(port)), timeout=1.0)
                    break
                except OSError as e:
                    if time.time() > deadline:
                        raise PeerTimeout(f"distributed.Init: rank {rank} could not reach coordinator "
                                          f"{peers[0]}: {e}") from None
                    time.sleep(0.02)
            c.settimeout(timeout)
            _tune(c)
            c.sendall(struct.pack(">II", MAGIC, rank))
            read_frame(c, OP_BARRIER, 0, "coordinator")
            self.conns = [c]

    # ---- accessors -----------------------------------------------------------------
    def Rank(self) -> int:
        return self.rank

    def WorldSize(self) -> int:
        return self.world

    def _alive(self):
        if self.closed:
            raise GroupClosed("collective on a closed group")

    # ---- collectives ------------------------------------------------------------------
    def _buf(self, name: str, n: int, dtype) -> np.ndarray:
        """A per-group scratch array, kept between collectives (a fresh 2 MB array per step costs more
        in page faults than the reduction itself)."""
        bufs = self.__dict__.setdefault("_bufs", {})
        b = bufs.get(name)
        if b is None or b.size != n or b.dtype != np.dtype(dtype):
            b = bufs[name] = np.empty(n, dtype=dtype)
        return b

    def _star(self, op: int, vec: np.ndarray, scale: float, own: bool = False) -> np.ndarray:
        """Gather to rank 0 in rank order, add, scale, send the same bytes back.  ``own``: ``vec`` is
        the caller's scratch and may be overwritten with the result."""
        self._alive()
        n = vec.size
        if self.world == 1:
            return vec * scale if scale != 1.0 else vec
        wire = self._buf("wire", n, ">f8") if n > 1024 else None
        if self.rank == 0:
            acc = vec if own and vec.dtype == np.float64 else np.array(vec, dtype=np.float64, copy=True)
            for r in range(1, self.world):
                acc += read_frame(self.conns[r], op, n, f"rank {r}", into=wire)
            if scale != 1.0:
                acc *= scale
            if wire is not None:
                wire[...] = acc                       # swap once, send the same bytes to everyone
            for r in range(1, self.world):
                if wire is not None:
                    write_frame(self.conns[r], op, acc, f"rank {r}", scratch=wire, prepared=True)
                else:
                    write_frame(self.conns[r], op, acc, f"rank {r}")
            return acc
        write_frame(self.conns[0], op, vec, "coordinator", scratch=wire)
        return read_frame(self.conns[0], op, n, "coordinator", into=wire)

    def AllReduceMeanGrads(self, params: Sequence[torch.Tensor]) -> None:
        """Mean of the flattened gradients over ranks; a missing gradient counts as zeros and
        is allocated on return (distributed.go:249-293)."""
        flat = self._buf("flat", sum(p.numel() for p in params), np.float64)
        off = 0
        for p in params:
            n = p.numel()
            if p.grad is None:
                flat[off:off + n] = 0.0
            else:
                t = p.grad.detach().cpu().reshape(-1)
                if t.dtype not in (torch.float64, torch.float32, torch.float16):
                    t = t.double()                                  # bfloat16 and integers have no numpy view
                flat[off:off + n] = t.numpy()                       # converts to float64 on assignment
            off += n
        out = self._star(OP_ALLREDUCE, flat, 1.0 / self.world, own=True)
        off = 0
        for p in params:
            n = p.numel()
            g = torch.from_numpy(out[off:off + n]).reshape(p.shape).to(dtype=p.dtype, device=p.device)
            if p.grad is None:
                p.grad = g.clone() if g.dtype == torch.float64 and g.device.type == "cpu" else g   # own storage
            else:
                p.grad.copy_(g)
            off += n

    all_reduce_mean_grads = AllReduceMeanGrads

    def AllReduceSum(self, vals: torch.Tensor) -> torch.Tensor:
        """In-place sum over ranks of a float vector (distributed.go:303-333)."""
        out = self._star(OP_ALLREDUCE_SUM, vals.detach().double().cpu().numpy().ravel(), 1.0)
        vals.copy_(torch.from_numpy(out.copy()).reshape(vals.shape).to(vals.dtype))
        return vals

    all_reduce_sum = AllReduceSum

    def BroadcastParams(self, params: Sequence[torch.Tensor], root: int = 0) -> None:
        """Every rank receives root's parameter values; a non-zero root relays through rank 0
        (distributed.go:338-388)."""
        self._alive()
        if self.world == 1:
            return
        n = sum(p.numel() for p in params)
        flat = None
        if self.rank == root:
            flat = np.concatenate([p.detach().double().cpu().numpy().ravel() for p in params])
        if root != 0:
            if self.rank == root:
                write_frame(self.conns[0], OP_BROADCAST, flat, "coordinator")
            elif self.rank == 0:
                flat = read_frame(self.conns[root], OP_BROADCAST, n, f"rank {root}")
        if self.rank == 0:
            for r in range(1, self.world):
                if r != root:
                    write_frame(self.conns[r], OP_BROADCAST, flat, f"rank {r}")
        elif self.rank != root:
            flat = read_frame(self.conns[0], OP_BROADCAST, n, "coordinator")
        off = 0
        with torch.no_grad():
            for p in params:
                k = p.numel()
                p.copy_(torch.from_numpy(flat[off:off + k].copy()).reshape(p.shape).to(p.dtype))
                off += k

    broadcast_params = BroadcastParams

    def Barrier(self) -> None:
        self._alive()
        if self.world == 1:
            return
        if self.rank == 0:
            for r in range(1, self.world):
                read_frame(self.conns[r], OP_BARRIER, 0, f"rank {r}")
            for r in range(1, self.world):
                write_frame(self.conns[r], OP_BARRIER, None, f"rank {r}")
        else:
            write_frame(self.conns[0], OP_BARRIER, None, "coordinator")
            read_frame(self.conns[0], OP_BARRIER, 0, "coordinator")

    barrier = Barrier

    def Close(self) -> None:
        self.closed = True
        for c in self.conns:
            if c is not None:
                try:
                    c.close()
                except OSError:
                    pass
        if self.lis is not None:
            try:
                self.lis.close()
            except OSError:
                pass
        self.conns = []

    close = Close


def Init(rank: int, world: int, peers: Sequence[str], timeout: float = 30.0) -> Group:
    """Connects the group; returns once every rank has joined (implicit barrier)."""
    return Group(rank, world, peers, timeout)


def DDPStep(group, opt) -> None:
    """All-reduce the mean gradients of the optimizer's parameters, then step
    (distributed.go:422-428)."""
    group.AllReduceMeanGrads(opt.parameters())
    opt.step()


def free_addr() -> str:
    """A localhost address with a currently free port (listen-and-close, like the
    reference's test helper)."""
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return f"127.0.0.1:{port}"

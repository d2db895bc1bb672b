"""CPU process group: the reference's distributed tests restated (distributed_test.go:20-320).
Ranks are threads that talk through real localhost TCP sockets; failure cases are made on
the host (a rank that never joins, closes mid-collective, calls a different collective, or is
slower than the deadline)."""
import socket
import struct
import threading
import time

import numpy as np
import pytest
import torch

from gonn_b200 import distributed as D
from gonn_b200 import optim
from gonn_b200.nn import Linear, Sequential, ReLU


def run_ranks(world, fn, timeout=10.0):
    addr = D.free_addr()
    out, errs = [None] * world, [None] * world

    def body(r):
        try:
            g = D.Init(r, world, [addr], timeout=timeout)
            try:
                out[r] = fn(g, r)
            finally:
                g.Close()
        except Exception as e:  # noqa: BLE001
            errs[r] = e

    ts = [threading.Thread(target=body, args=(r,)) for r in range(world)]
    [t.start() for t in ts]
    [t.join(60) for t in ts]
    return out, errs


def test_mean_grads_with_missing_grad():
    def fn(g, r):
        a = torch.nn.Parameter(torch.zeros(3, dtype=torch.float64))
        b = torch.nn.Parameter(torch.zeros(2, dtype=torch.float64))
        a.grad = torch.tensor([1.0, 2.0, 3.0], dtype=torch.float64) * (r + 1)
        if r != 1:
            b.grad = torch.tensor([10.0, 20.0], dtype=torch.float64)
        g.AllReduceMeanGrads([a, b])
        return a.grad.clone(), b.grad.clone()

    out, errs = run_ranks(3, fn)
    assert errs == [None] * 3
    for a, b in out:
        assert torch.equal(a, torch.tensor([2.0, 4.0, 6.0], dtype=torch.float64))
        assert torch.allclose(b, torch.tensor([20.0 / 3, 40.0 / 3], dtype=torch.float64), atol=1e-15)
    assert all(torch.equal(out[0][1], o[1]) for o in out)  # bit-identical on every rank


@pytest.mark.parametrize("root", [0, 2])
def test_broadcast_direct_and_relayed(root):
    def fn(g, r):
        p = torch.nn.Parameter(torch.full((4,), float(r), dtype=torch.float64))
        g.BroadcastParams([p], root)
        return p.detach().clone()

    out, errs = run_ranks(3, fn)
    assert errs == [None] * 3
    assert all(torch.equal(o, torch.full((4,), float(root), dtype=torch.float64)) for o in out)


def test_barrier_and_sum():
    order = []

    def fn(g, r):
        time.sleep(0.05 * r)
        order.append(("before", r))
        g.Barrier()
        order.append(("after", r))
        v = torch.tensor([1.0, float(r)], dtype=torch.float64)
        g.AllReduceSum(v)
        return v

    out, errs = run_ranks(3, fn)
    assert errs == [None] * 3
    firsts = [i for i, (k, _) in enumerate(order) if k == "after"]
    lasts = [i for i, (k, _) in enumerate(order) if k == "before"]
    assert min(firsts) > max(lasts)
    assert all(torch.equal(o, torch.tensor([3.0, 3.0], dtype=torch.float64)) for o in out)


def test_world_one_is_a_no_op():
    g = D.Init(0, 1, ["127.0.0.1:1"])
    p = torch.nn.Parameter(torch.ones(2, dtype=torch.float64))
    p.grad = torch.tensor([3.0, 4.0], dtype=torch.float64)
    g.AllReduceMeanGrads([p])
    g.BroadcastParams([p], 0)
    g.Barrier()
    assert torch.equal(p.grad, torch.tensor([3.0, 4.0], dtype=torch.float64))
    g.Close()


_PROTO = []


def _model():
    # the global generator is shared by the rank threads: build once, hand out copies
    import copy
    if not _PROTO:
        torch.manual_seed(7)
        _PROTO.append(Sequential(Linear(6, 5, dtype=torch.float64), ReLU(), Linear(5, 3, dtype=torch.float64)))
    return copy.deepcopy(_PROTO[0])


def test_two_rank_ddp_equals_full_batch():
    """Equal shards + mean loss: the data-parallel run equals the full-batch run to 1e-12 and
    the ranks stay bit-identical (distributed_test.go:205-277)."""
    torch.manual_seed(3)
    X = torch.randn(8, 6, dtype=torch.float64)
    Y = torch.randn(8, 3, dtype=torch.float64)
    ref = _model()
    opt = optim.SGD(ref.parameters(), lr=0.1, momentum=0.9)
    for _ in range(5):
        opt.zero_grad()
        ((ref(X) - Y) ** 2).mean().backward()
        opt.step()

    def fn(g, r):
        m = _model()
        g.BroadcastParams(list(m.parameters()), 0)
        o = optim.SGD(m.parameters(), lr=0.1, momentum=0.9)
        xs, ys = X[r * 4:(r + 1) * 4], Y[r * 4:(r + 1) * 4]
        for _ in range(5):
            o.zero_grad()
            ((m(xs) - ys) ** 2).mean().backward()
            D.DDPStep(g, o)
        return [p.detach().clone() for p in m.parameters()]

    out, errs = run_ranks(2, fn)
    assert errs == [None, None]
    for p0, p1, pr in zip(out[0], out[1], ref.parameters()):
        assert torch.equal(p0, p1)
        assert (p0 - pr).abs().max().item() < 1e-12


def test_protocol_mismatch_detected():
    def fn(g, r):
        v = torch.zeros(3, dtype=torch.float64)
        if r == 0:
            g.AllReduceSum(v)
        else:
            g.Barrier()

    _, errs = run_ranks(2, fn, timeout=3.0)
    assert any(isinstance(e, D.ProtocolError) for e in errs)


def test_count_mismatch_detected():
    def fn(g, r):
        g.AllReduceSum(torch.zeros(3 + r, dtype=torch.float64))

    _, errs = run_ranks(2, fn, timeout=3.0)
    assert any(isinstance(e, (D.ProtocolError, D.PeerClosed, D.PeerTimeout)) for e in errs)
    assert any(isinstance(e, D.ProtocolError) for e in errs)


def test_rank_never_joins_times_out(monkeypatch):
    monkeypatch.setattr(D.tcp, "DialTimeout", 0.5)
    addr = D.free_addr()
    t0 = time.time()
    with pytest.raises(D.PeerTimeout):
        D.Init(0, 2, [addr], timeout=0.5)
    assert time.time() - t0 < 5
    with pytest.raises(D.PeerTimeout):
        D.Init(1, 2, [D.free_addr()], timeout=0.5)


def test_peer_closes_mid_collective():
    def fn(g, r):
        if r == 1:
            g.Close()
            return None
        time.sleep(0.1)
        g.AllReduceSum(torch.zeros(4, dtype=torch.float64))

    _, errs = run_ranks(2, fn, timeout=2.0)
    assert isinstance(errs[0], (D.PeerClosed, D.PeerTimeout))


def test_slow_peer_hits_deadline():
    def fn(g, r):
        if r == 1:
            time.sleep(1.5)
        g.AllReduceSum(torch.zeros(4, dtype=torch.float64))

    _, errs = run_ranks(2, fn, timeout=0.4)
    assert isinstance(errs[0], D.PeerTimeout)


def test_bad_magic_and_duplicate_rank_rejected():
    addr = D.free_addr()
    host, port = addr.split(":")
    err = {}

    def coord():
        try:
            D.Init(0, 2, [addr], timeout=2.0)
        except Exception as e:  # noqa: BLE001
            err["e"] = e

    t = threading.Thread(target=coord)
    t.start()
    time.sleep(0.2)
    c = socket.create_connection((host, int(port)))
    c.sendall(struct.pack(">II", 0xDEADBEEF, 1))
    t.join(5)
    c.close()
    assert isinstance(err.get("e"), D.ProtocolError)


def test_closed_group_raises():
    g = D.Init(0, 1, ["127.0.0.1:1"])
    g.Close()
    with pytest.raises(D.GroupClosed):
        g.Barrier()


def test_wire_frame_layout():
    a, b = socket.socketpair()
    D.tcp.write_frame(a, D.tcp.OP_ALLREDUCE_SUM, np.array([1.5, -2.0]))
    raw = b.recv(64)
    assert raw[0] == 4 and struct.unpack(">Q", raw[1:9])[0] == 2
    assert struct.unpack(">dd", raw[9:25]) == (1.5, -2.0)
    a.close(); b.close()


def test_large_frames_reuse_scratch_arrays_and_keep_the_wire_format():
    """Frames above 1024 elements go out of, and come into, persistent big-endian arrays: the bytes
    on the wire stay ``[op][count][count x big-endian float64]`` and a second collective through the
    same arrays is not polluted by the first."""
    n = 5000
    a, b = socket.socketpair()
    a.settimeout(5); b.settimeout(5)
    vals = np.arange(n, dtype=np.float64) * 0.5 - 7
    scratch = np.empty(n, dtype=">f8")
    got = {}

    def reader():
        got["raw"] = D.tcp._recv_exact(b, 9 + 8 * n, "peer")

    t = threading.Thread(target=reader); t.start()
    D.tcp.write_frame(a, D.tcp.OP_ALLREDUCE, vals, scratch=scratch)
    t.join(10)
    raw = got["raw"]
    assert raw[0] == 1 and struct.unpack(">Q", raw[1:9])[0] == n
    assert np.array_equal(np.frombuffer(raw[9:], dtype=">f8").astype(np.float64), vals)
    # the receiving side, twice into the same array
    into = np.empty(n, dtype=">f8")
    for k in (1.0, -3.0):
        t = threading.Thread(target=lambda: D.tcp.write_frame(a, D.tcp.OP_ALLREDUCE, vals * k)); t.start()
        out = D.tcp.read_frame(b, D.tcp.OP_ALLREDUCE, n, into=into)
        t.join(10)
        assert out.dtype == np.float64 and np.array_equal(out, vals * k)
    a.close(); b.close()

    # and through a group: two all-reduces of 3000 gradients each give exact means both times
    def fn(g, r):
        p = torch.zeros(3000, dtype=torch.float64, requires_grad=True)
        res = []
        for step in range(2):
            p.grad = torch.full((3000,), float(r + 1 + 10 * step), dtype=torch.float64)
            g.AllReduceMeanGrads([p])
            res.append(p.grad.clone())
        return res

    out, errs = run_ranks(2, fn)
    assert errs == [None, None]
    for r in range(2):
        assert torch.equal(out[r][0], torch.full((3000,), 1.5, dtype=torch.float64))
        assert torch.equal(out[r][1], torch.full((3000,), 11.5, dtype=torch.float64))


def test_mean_grads_of_bfloat16_and_float32_parameters():
    def fn(g, r):
        a = torch.zeros(5, dtype=torch.bfloat16, requires_grad=True)
        b = torch.zeros(3, dtype=torch.float32, requires_grad=True)
        a.grad = torch.full((5,), float(r + 1), dtype=torch.bfloat16)
        b.grad = torch.full((3,), float(2 * r), dtype=torch.float32)
        g.AllReduceMeanGrads([a, b])
        return a.grad, b.grad

    out, errs = run_ranks(2, fn)
    assert errs == [None, None]
    for ga, gb in out:
        assert ga.dtype == torch.bfloat16 and torch.equal(ga.float(), torch.full((5,), 1.5))
        assert gb.dtype == torch.float32 and torch.equal(gb, torch.full((3,), 1.0))

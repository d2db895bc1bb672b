"""Checkpoint round trips, in-process DataParallel, backend contract, tensor API, data loader,
data-parallel engine on the host oracle path."""
import numpy as np
import pytest
import torch

from gonn_b200 import backend, data, nn, optim, parallel
from gonn_b200 import tensor as T
from gonn_b200.models import MLP, TransformerLM
from gonn_b200.utils import checkpoint


def test_checkpoint_round_trip_and_cross_dtype(tmp_path):
    torch.manual_seed(0)
    m = nn.Sequential(nn.Linear(4, 3, dtype=torch.float64), nn.BatchNorm1d(3, dtype=torch.float64))
    o = optim.Adam(m.parameters(), lr=0.1)
    x = torch.randn(5, 4, dtype=torch.float64)
    for _ in range(3):
        o.zero_grad(); m(x).pow(2).sum().backward(); o.step()
    p = str(tmp_path / "a.ckpt")
    checkpoint.save(p, m, o)
    ent = checkpoint.read(p)
    assert list(ent)[:4] == ["0.weight", "0.bias", "1.weight", "1.bias"]
    assert "1.running_mean" in ent and "0.weight/m" in ent and "@opt/t" in ent
    m2 = nn.Sequential(nn.Linear(4, 3, dtype=torch.float64), nn.BatchNorm1d(3, dtype=torch.float64))
    o2 = optim.Adam(m2.parameters(), lr=0.5)
    checkpoint.load(p, m2, o2)
    for a, b in zip(m.state_dict().values(), m2.state_dict().values()):
        assert torch.equal(a, b)                 # fp64 payload is exact
    assert o2.t == o.t and o2.lr() == 0.1
    # resumed training equals uninterrupted training
    for mm, oo in ((m, o), (m2, o2)):
        oo.zero_grad(); mm(x).pow(2).sum().backward(); oo.step()
    assert torch.equal(m[0].weight, m2[0].weight)
    m3 = nn.Sequential(nn.Linear(4, 3, dtype=torch.bfloat16), nn.BatchNorm1d(3, dtype=torch.bfloat16))
    checkpoint.load(p, m3)
    assert (m3[0].weight.double() - ent["0.weight"][1]).abs().max().item() < 1e-2
    with open(p, "rb") as f:
        assert f.read(8) == b"GONNCKPT"
    (tmp_path / "bad").write_bytes(b"nonsense")
    with pytest.raises(ValueError):
        checkpoint.read(str(tmp_path / "bad"))


def test_data_parallel_equals_full_batch():
    torch.manual_seed(0)
    X, Y = torch.randn(10, 4, dtype=torch.float64), torch.randn(10, 2, dtype=torch.float64)
    ref = nn.Linear(4, 2, dtype=torch.float64)
    par = nn.Linear(4, 2, dtype=torch.float64)
    par.load_state_dict(ref.state_dict())
    o1, o2 = optim.SGD(ref.parameters(), lr=0.1), optim.SGD(par.parameters(), lr=0.1)
    o1.zero_grad(); ((ref(X) - Y) ** 2).mean().backward(); o1.step()
    loss = parallel.DataParallel(3).step(o2, lambda x, y: ((par(x) - y) ** 2).mean(), X, Y)
    assert (ref.weight - par.weight).abs().max().item() < 1e-12
    assert parallel.shard_bounds(10, 3) == [(0, 4), (4, 7), (7, 10)]
    assert loss == pytest.approx(float(((ref(X) - Y) ** 2).mean().detach()), abs=1.0)


def test_backend_contract_and_fake():
    class Fake(backend.Backend):
        calls = 0

        def Name(self): return "fake"

        def Gemm(self, a, b, batch, m, k, n, transA=False, transB=False):
            Fake.calls += 1
            return torch.zeros(batch, m, n)
    prev = backend.Use(Fake())
    assert backend.Current().Name() == "fake" and backend.Current().Gemm(None, None, 1, 2, 3, 4).shape == (1, 2, 4)
    backend.Use(prev)
    cpu = backend.NewCPU()
    a, b = torch.randn(2, 3, 4, dtype=torch.float64), torch.randn(2, 5, 4, dtype=torch.float64)
    out = cpu.Gemm(a, b, 2, 3, 4, 5, False, True)
    assert (out - a @ b.transpose(1, 2)).abs().max().item() < 1e-12
    assert int(backend.UnaryKind.GELUExact) == 7 and int(backend.BinaryKind.Div) == 3
    assert not hasattr(backend.Backend, "Unary")      # the elementwise capability is optional


def test_tensor_api():
    x = T.New([1.0, 2.0, 3.0, 4.0, 5.0, 6.0], 2, 3, requires_grad=True)
    y = T.Sum(T.Mul(T.Exp(x), T.Full(2.0, 2, 3)))
    T.Backward(y)
    assert (x.grad - 2 * torch.exp(x.detach())).abs().max().item() < 1e-12
    assert len(T.UnaryOpNames()) == 25 and T.LookupUnary("relu").Kind == 9 and T.LookupUnary("nope") is None
    with pytest.raises(ValueError):
        T.RegisterUnary(T.UnaryOpDef("relu", lambda a: a, lambda a, g: g))
    T.RegisterUnary(T.UnaryOpDef("cube_test", lambda a: a ** 3, lambda a, g: 3 * a * a * g))
    z = x.detach().clone().requires_grad_(True)
    T.Sum(T.Unary(z, "cube_test")).backward()
    assert (z.grad - 3 * z.detach() ** 2).abs().max().item() < 1e-12
    assert T.ArgMax(T.New([1.0, 3.0, 3.0], 1, 3), 1).tolist() == [1]          # first maximum wins
    assert T.MatMul(T.Ones(2, 3), T.Ones(3, 4)).shape == (2, 4)
    assert T.BMM(T.Ones(2, 2, 3), T.Ones(2, 3, 1)).shape == (2, 2, 1)
    with pytest.raises(ValueError):
        T.BMM(T.Ones(2, 2, 3), T.Ones(3, 3, 1))
    assert T.RoundTo(T.New([1.0 + 2 ** -12]), torch.float16).item() == 1.0
    mn = T.MakeNode(lambda a: a * 2, "Double", [z], lambda g: [g * 2])
    mn.sum().backward()
    old = T.SetDispatchPolicy(T.DispatchPolicy(0, 0))
    assert old.UnaryMinElems == 1 << 16 and T.GetDispatchPolicy().UnaryMinElems == 0
    T.SetDispatchPolicy(old)
    assert T.BroadcastShapes((3, 1), (4,)) == (3, 4)
    w = T.Where(T.New([1.0, 0.0]) > 0, T.New([5.0, 5.0]), 7.0)
    assert w.tolist() == [5.0, 7.0]


def test_data_loader_and_transforms(tmp_path):
    X, y = data.MakeClassification(20, 3, 2, seed=1)
    ds = data.TensorDataset(X, y)
    a, _ = ds.Get(0)
    a += 100
    assert ds.Get(0)[0][0] < 50                       # Get returns a deep copy
    dl = data.DataLoader(ds, 6, shuffle=True, drop_last=True, seed=3)
    b1 = [yb.tolist() for _, yb in dl.Iter()]
    assert len(b1) == 3 == len(dl)
    img = torch.arange(2 * 4 * 4, dtype=torch.float32).reshape(2, 4, 4)
    t = data.Compose(data.Normalize([0.0, 1.0], [1.0, 2.0]), data.RandomCrop(2, seed=0), data.RandomHorizontalFlip(1.0))
    assert t(img).shape == (2, 2, 2)
    csvp = tmp_path / "d.csv"
    csvp.write_text("a,b,y\n1,2,3\n4,5,6\n")
    c = data.LoadCSV(str(csvp))
    assert c.X.tolist() == [[1.0, 2.0], [4.0, 5.0]] and c.Y.tolist() == [3.0, 6.0]
    Xm, ym = data.MakeMoons(50)
    assert Xm.shape == (50, 2) and set(ym.tolist()) == {0, 1}
    with pytest.raises(FileNotFoundError):
        data.LoadMNIST(str(tmp_path))


def test_engine_host_path_matches_plain_adamw():
    from gonn_b200.distributed.ddp import DistributedDataParallel
    torch.manual_seed(0)
    kw = dict(vocab=64, d_model=32, n_layers=1, n_heads=2, d_ff=64, max_seq=16, dtype=torch.bfloat16)
    a, b = TransformerLM(**kw), TransformerLM(**kw)
    b.load_state_dict(a.state_dict())
    ddp = DistributedDataParallel(a, optimizer=dict(kind="adamw", lr=1e-2, weight_decay=0.1), bucket_mb=0.01)
    assert len(ddp.buckets) > 1
    opt = optim.AdamW(b.parameters(), lr=1e-2, weight_decay=0.1)
    ids = torch.randint(0, 64, (2, 16))
    for _ in range(3):
        a.loss(ids, ids).backward(); ddp.step()
        opt.zero_grad(); b.loss(ids, ids).backward(); opt.step()
    for (n, p), q in zip(a.named_parameters(), b.parameters()):
        assert (p.float() - q.float()).abs().max().item() < 2e-2, n
    with ddp.no_sync():
        a.loss(ids, ids).backward()
    g1 = ddp.flat_grads.clone()
    a.loss(ids, ids).backward()
    assert (ddp.flat_grads.float() - 2 * g1.float()).abs().max().item() < 0.05   # accumulated
    ddp.step()


def test_mlp_config1_trains_on_cpu():
    torch.manual_seed(0)
    m = MLP((784, 256, 128, 10))
    o = optim.SGD(m.parameters(), lr=0.01, momentum=0.9)
    x, y = torch.rand(64, 1, 28, 28), torch.randint(0, 10, (64,))
    l0 = None
    for _ in range(250):
        o.zero_grad()
        loss = nn.CrossEntropyLoss(m(x), y)
        loss.backward()
        o.step()
        l0 = l0 or loss.item()
    assert loss.item() < l0 - 0.3

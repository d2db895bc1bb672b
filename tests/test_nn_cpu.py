"""Module system contracts: naming, order, registration completeness, gradcheck harness over
the layer catalogue (nn/module_test.go, nn/gradcheck_test.go, nn/parity_test.go patterns)."""
import math

import pytest
import torch

from gonn_b200 import nn
from gonn_b200.models import TransformerLM


def gradcheck(fn, inputs, eps=1e-5, rtol=1e-4, max_elems=24, seed=0):
    """Central differences with optional sampling of ``max_elems`` indices per input."""
    g = torch.Generator().manual_seed(seed)
    for x in inputs:
        x.grad = None
    fn().backward()
    for x in inputs:
        ana = x.grad.clone() if x.grad is not None else torch.zeros_like(x)
        idx = torch.randperm(x.numel(), generator=g)[:max_elems]
        flat = x.data.reshape(-1)
        for i in idx.tolist():
            old = float(flat[i])
            flat[i] = old + eps
            up = float(fn())
            flat[i] = old - eps
            dn = float(fn())
            flat[i] = old
            num = (up - dn) / (2 * eps)
            a = float(ana.reshape(-1)[i])
            assert abs(a - num) <= rtol * max(1.0, abs(a), abs(num)), (i, a, num)


D = torch.float64


def _w(shape):
    return torch.randn(shape, dtype=D)


LAYERS = [
    ("Linear", lambda: nn.Linear(5, 4, dtype=D), (3, 5)),
    ("Conv1d", lambda: nn.Conv1d(2, 3, 3, padding=1, dtype=D), (2, 2, 7)),
    ("Conv2d", lambda: nn.Conv2d(2, 3, 3, stride=2, padding=1, dtype=D), (2, 2, 6, 5)),
    ("Conv3d", lambda: nn.Conv3d(1, 2, 2, dtype=D), (1, 1, 3, 4, 3)),
    ("ConvTranspose2d", lambda: nn.ConvTranspose2d(2, 3, 3, stride=2, dtype=D), (1, 2, 3, 3)),
    ("MaxPool2d", lambda: nn.MaxPool2d(2), (1, 2, 4, 6)),
    ("AvgPool2d", lambda: nn.AvgPool2d(2, 1, 1), (1, 2, 4, 4)),
    ("AdaptiveAvgPool2d", lambda: nn.AdaptiveAvgPool2d((2, 3)), (1, 2, 5, 7)),
    ("LayerNorm", lambda: nn.LayerNorm(6, dtype=D), (4, 6)),
    ("RMSNorm", lambda: nn.RMSNorm(6, dtype=D), (4, 6)),
    ("GroupNorm", lambda: nn.GroupNorm(2, 4, dtype=D), (2, 4, 3)),
    ("InstanceNorm2d", lambda: nn.InstanceNorm2d(3), (2, 3, 4, 4)),
    ("BatchNorm1d", lambda: nn.BatchNorm1d(4, dtype=D), (6, 4)),
    ("BatchNorm2d", lambda: nn.BatchNorm2d(3, dtype=D), (4, 3, 3, 2)),
    ("PReLU", lambda: nn.PReLU(dtype=D), (3, 4)),
    ("GLU", lambda: nn.GLU(), (3, 6)),
    ("GELU", lambda: nn.GELU(), (3, 4)),
    ("SiLU", lambda: nn.SiLU(), (3, 4)),
    ("Mish", lambda: nn.Mish(), (3, 4)),
    ("ELU", lambda: nn.ELU(1.3), (3, 4)),
    ("Softplus", lambda: nn.Softplus(), (3, 4)),
    ("Tanh", lambda: nn.Tanh(), (3, 4)),
    ("Softmax", lambda: nn.Softmax(-1), (3, 5)),
    ("LogSoftmax", lambda: nn.LogSoftmax(-1), (3, 5)),
    ("ReflectionPad2d", lambda: nn.ReflectionPad2d(1), (1, 2, 3, 4)),
    ("Upsample", lambda: nn.Upsample(2, "bilinear"), (1, 2, 3, 3)),
    ("LocalResponseNorm", lambda: nn.LocalResponseNorm(3), (2, 4, 3)),
]


@pytest.mark.parametrize("name,make,shape", LAYERS, ids=[l[0] for l in LAYERS])
def test_gradcheck_layers(name, make, shape):
    torch.manual_seed(1)
    m = make()
    x = _w(shape).requires_grad_(True)
    w = _w(m(x).shape)
    params = [x] + [p for p in m.parameters()]
    gradcheck(lambda: (m(x) * w).sum(), params)


def test_gradcheck_attention_rnn_losses():
    torch.manual_seed(2)
    mha = nn.MultiHeadAttention(8, 2, dtype=D)
    x = _w((2, 5, 8)).requires_grad_(True)
    w = _w((2, 5, 8))
    gradcheck(lambda: (mha(x, x, x, True) * w).sum(), [x] + list(mha.parameters()), max_elems=10)
    for cls in (nn.RNN, nn.LSTM, nn.GRU):
        r = cls(3, 4, num_layers=2, bidirectional=True, dtype=D)
        xs = _w((2, 4, 3)).requires_grad_(True)
        ww = _w((2, 4, 8))
        gradcheck(lambda: (r(xs) * ww).sum(), [xs] + list(r.parameters()), max_elems=6)
    logits = _w((6, 5)).requires_grad_(True)
    t = torch.randint(0, 5, (6,))
    wts = torch.rand(5, dtype=D) + 0.5
    gradcheck(lambda: nn.CrossEntropyLoss(logits, t, weight=wts, label_smoothing=0.1, ignore_index=2), [logits])
    p, q = _w((4, 3)).requires_grad_(True), _w((4, 3))
    gradcheck(lambda: nn.HuberLoss(p, q, 0.7), [p])
    gradcheck(lambda: nn.BCEWithLogitsLoss(p, (q > 0).to(D)), [p])
    gradcheck(lambda: nn.TripletMarginLoss(p, q, q.flip(0)), [p])
    lp = _w((7, 2, 4)).log_softmax(2).detach().requires_grad_(True)
    gradcheck(lambda: nn.CTCLoss(lp, torch.tensor([[1, 2], [3, 1]]), [7, 6], [2, 2]), [lp], max_elems=12)


def test_state_dict_names():
    """Parameter / buffer names of the reference (its naming contract for checkpoints)."""
    enc = nn.TransformerEncoderLayer(8, 2, 16)
    names = [n for n, _ in enc.named_parameters()]
    assert names == ["attn.qproj.weight", "attn.qproj.bias", "attn.kproj.weight", "attn.kproj.bias",
                     "attn.vproj.weight", "attn.vproj.bias", "attn.outproj.weight", "attn.outproj.bias",
                     "norm1.weight", "norm1.bias", "ff1.weight", "ff1.bias", "ff2.weight", "ff2.bias",
                     "norm2.weight", "norm2.bias"]
    dec = nn.TransformerDecoderLayer(8, 2, 16)
    assert [n.split(".")[0] for n, _ in dec.named_children()] == [
        "selfattn", "norm1", "crossattn", "norm2", "ff1", "ff2", "norm3", "act", "drop1", "drop2", "drop3", "dropff"]
    tr = nn.Transformer(8, 2, 1, 1, 16)
    assert {n.split(".")[0] for n, _ in tr.named_parameters()} == {"encoder", "decoder", "encnorm", "decnorm"}
    assert any(n.startswith("encoder.layers.0.attn.") for n, _ in tr.named_parameters())
    seq = nn.Sequential(nn.Linear(2, 3), nn.ReLU(), nn.Linear(3, 1))
    assert [n for n, _ in seq.named_parameters()] == ["0.weight", "0.bias", "2.weight", "2.bias"]
    bn = nn.BatchNorm2d(3)
    assert [n for n, _ in bn.named_buffers()] == ["running_mean", "running_var"]   # no num_batches_tracked
    lstm = nn.LSTM(3, 4, num_layers=2, bidirectional=True, proj_size=2)
    ns = [n for n, _ in lstm.named_parameters()]
    assert "cells.0.wih.weight" in ns and "backcells.1.whh.weight" in ns and "cells.0.whr.weight" in ns
    s2s = nn.Seq2Seq(10, 12, 4, 6)
    assert [n for n, _ in s2s.named_children()] == ["embsrc", "embtgt", "encoder", "decoder", "outproj"]
    md = nn.ModuleDict({"b": nn.Linear(1, 1), "a": nn.Linear(1, 1)})
    assert md.Keys() == ["a", "b"]


def test_registration_completeness():
    """Every tensor that requires grad and is reachable from a module attribute is in parameters()."""
    model = TransformerLM(vocab=32, d_model=16, n_layers=2, n_heads=2, d_ff=32, max_seq=8)
    reg = {id(p) for p in model.parameters()}
    seen = set()

    def walk(obj):
        if id(obj) in seen:
            return
        seen.add(id(obj))
        if isinstance(obj, torch.Tensor):
            if obj.requires_grad and obj.is_leaf:
                assert id(obj) in reg
            return
        if isinstance(obj, torch.nn.Module):
            for v in list(vars(obj).values()) + list(obj._parameters.values()) + list(obj._modules.values()):
                walk(v)
        elif isinstance(obj, (list, tuple)):
            for v in obj:
                walk(v)
        elif isinstance(obj, dict):
            for v in obj.values():
                walk(v)
    walk(model)
    assert len(reg) == len(list(model.parameters()))


def test_init_distribution_and_conventions():
    torch.manual_seed(0)
    l = nn.Linear(400, 300)
    b = math.sqrt(1 / 400)
    assert l.weight.abs().max().item() <= b and l.bias.abs().max().item() <= b
    assert abs(l.weight.std().item() - b / math.sqrt(3)) < 0.1 * b
    assert nn.Embedding(1000, 64).weight.std().item() == pytest.approx(1.0, abs=0.05)
    assert nn.PReLU().weight.item() == 0.25
    x = torch.linspace(-3, 3, 13, dtype=D)
    assert (nn.GELU()(x) - torch.nn.functional.gelu(x, approximate="tanh")).abs().max().item() < 1e-12
    assert (nn.GELUExact()(x) - torch.nn.functional.gelu(x)).abs().max().item() < 1e-12
    big = torch.tensor([25.0], dtype=D)
    assert nn.Softplus()(big).item() == 25.0                       # linear above 20
    r = nn.RMSNorm(4, dtype=D)
    v = torch.tensor([[1.0, 2.0, 3.0, 4.0]], dtype=D)
    assert (r(v) - v / torch.sqrt((v * v).mean() + 1e-6)).abs().max().item() < 1e-12


def test_hooks_functional_call_and_train_flag():
    lin = nn.Linear(3, 2, dtype=D)
    calls = []
    h1 = nn.RegisterForwardPreHook(lin, lambda m, x: x * 2)
    h2 = nn.RegisterForwardHook(lin, lambda m, x, y: calls.append("fwd") or None)
    h3 = nn.RegisterFullBackwardHook(lin, lambda m, g: calls.append("bwd") or None)
    x = torch.ones(1, 3, dtype=D, requires_grad=True)
    y = nn.Call(lin, x)
    assert torch.allclose(y, lin.forward(x * 2))
    y.sum().backward()
    assert calls == ["fwd", "bwd"]
    assert nn.RemoveHook(h1) and nn.RemoveHook(h2) and nn.RemoveHook(h3) and not nn.RemoveHook(h1)
    rep = {"weight": torch.zeros(2, 3, dtype=D), "bias": torch.ones(2, dtype=D)}
    assert torch.equal(nn.FunctionalCall(lin, x, rep), torch.ones(1, 2, dtype=D))
    before = lin.weight.detach().clone()
    with nn.WithReplacedParams(lin, rep):
        assert torch.equal(lin.weight.data, rep["weight"])
    assert torch.equal(lin.weight.data, before)
    loss, grads = nn.FunctionalCallGrad(lin, x, rep, lambda out: out.sum())
    assert grads["bias"].tolist() == [1.0, 1.0]
    seq = nn.Sequential(nn.Dropout(0.5), nn.BatchNorm1d(3))
    assert seq.Training and seq[0].training
    seq.Eval()
    assert not seq[1].training and torch.equal(seq[0](x), x)
    assert [id(p) for p in nn.FilterParams(seq, lambda n, p: n.endswith("bias"))] == [id(seq[1].bias)]


def test_feed_forward_matches_composed_layers():
    """The fused two-layer node must give the gradients of the composed expression."""
    from gonn_b200.ops.linear import feed_forward
    torch.manual_seed(3)
    for act, ref in (("gelu", lambda t: torch.nn.functional.gelu(t, approximate="tanh")),
                     ("relu", torch.relu),
                     ("geluexact", torch.nn.functional.gelu)):
        x = torch.randn(5, 7, 12, dtype=torch.float64, requires_grad=True)
        w1 = torch.randn(20, 12, dtype=torch.float64, requires_grad=True)
        b1 = torch.randn(20, dtype=torch.float64, requires_grad=True)
        w2 = torch.randn(12, 20, dtype=torch.float64, requires_grad=True)
        b2 = torch.randn(12, dtype=torch.float64, requires_grad=True)
        res = torch.randn(5, 7, 12, dtype=torch.float64, requires_grad=True)
        y = feed_forward(x, w1, b1, w2, b2, act, res)
        g = torch.randn_like(y)
        got = torch.autograd.grad(y, (x, w1, b1, w2, b2, res), g)
        yr = ref(x @ w1.t() + b1) @ w2.t() + b2 + res
        want = torch.autograd.grad(yr, (x, w1, b1, w2, b2, res), g)
        assert torch.allclose(y, yr, atol=1e-9)
        for a, b in zip(got, want):
            assert torch.allclose(a, b, atol=1e-8), act


def test_functional_call_grads_to_replacements():
    import gonn_b200.nn as gnn
    torch.manual_seed(0)
    lin = gnn.Linear(4, 3, dtype=torch.float64)
    x = torch.randn(5, 4, dtype=torch.float64)
    w2 = torch.randn(3, 4, dtype=torch.float64)
    loss, grads = gnn.FunctionalCallGrad(lin, x, {"weight": w2}, lambda y: (y ** 2).mean(),
                                         gnn.WithGradsToReplacements())
    assert set(grads) == {"weight"} and lin.weight.grad is None
    assert torch.allclose(w2.grad, grads["weight"])
    # a second call accumulates
    gnn.FunctionalCallGrad(lin, x, {"weight": w2}, lambda y: (y ** 2).mean(), gnn.WithGradsToReplacements())
    assert torch.allclose(w2.grad, 2 * grads["weight"])
    assert gnn.ParametrizationWithInverse is gnn.InvertibleParametrization


def test_lstm_gru_cells_match_torch_cells():
    """Cell formulas (gate order i,f,g,o / r,z,n) against torch's cells with copied weights."""
    import gonn_b200.nn as gnn
    torch.manual_seed(0)
    x = torch.randn(5, 7, dtype=torch.float64)
    h = torch.randn(5, 6, dtype=torch.float64)
    c = torch.randn(5, 6, dtype=torch.float64)
    mine = gnn.LSTMCell(7, 6, dtype=torch.float64)
    ref = torch.nn.LSTMCell(7, 6, dtype=torch.float64)
    with torch.no_grad():
        ref.weight_ih.copy_(mine.wih.weight); ref.bias_ih.copy_(mine.wih.bias)
        ref.weight_hh.copy_(mine.whh.weight); ref.bias_hh.zero_()
    h1, c1 = mine(x, (h, c))
    h2, c2 = ref(x, (h, c))
    assert torch.allclose(h1, h2, atol=1e-10) and torch.allclose(c1, c2, atol=1e-10)
    g1 = gnn.GRUCell(7, 6, dtype=torch.float64)
    g2 = torch.nn.GRUCell(7, 6, dtype=torch.float64)
    with torch.no_grad():
        g2.weight_ih.copy_(g1.wih.weight); g2.bias_ih.copy_(g1.wih.bias)
        g2.weight_hh.copy_(g1.whh.weight); g2.bias_hh.copy_(g1.whh.bias)
    assert torch.allclose(g1(x, h), g2(x, h), atol=1e-10)

"""Semantics tests in the style of the reference's: packed sequences equal per-sequence runs,
convolution / pooling options against torch's layers, concurrent backward into shared leaves
with integer-valued gradients, whole-stack RNNs against torch's."""
import threading

import pytest
import torch
import torch.nn.functional as F

from gonn_b200 import nn

D = torch.float64


def _x(*shape, seed=0):
    return torch.randn(*shape, dtype=D, generator=torch.Generator().manual_seed(seed))


@pytest.mark.parametrize("kind", ["rnn", "lstm", "gru"])
@pytest.mark.parametrize("bidir", [False, True])
def test_packed_batch_equals_per_sequence_runs(kind, bidir):
    torch.manual_seed(0)
    cls = {"rnn": nn.RNN, "lstm": nn.LSTM, "gru": nn.GRU}[kind]
    m = cls(3, 4, num_layers=2, bidirectional=bidir, dtype=D)
    seqs = [_x(5, 3, seed=1), _x(2, 3, seed=2), _x(4, 3, seed=3)]
    packed = nn.PackSequence(seqs)
    out, st = m.ForwardPacked(packed)
    padded, lengths = nn.PadPackedSequence(out)
    assert lengths == [5, 2, 4] and padded.shape == (3, 5, 4 * (2 if bidir else 1))
    h = st[0] if kind == "lstm" else st
    for b, s in enumerate(seqs):
        o1, s1 = m.ForwardWithState(s[None])
        assert torch.allclose(padded[b, :len(s)], o1[0], rtol=0, atol=1e-14), (kind, bidir, b)
        assert bool((padded[b, len(s):] == 0).all())                # padding steps produce nothing
        h1 = s1[0] if kind == "lstm" else s1
        assert torch.allclose(h[:, b], h1[:, 0], rtol=0, atol=1e-14)  # ... and do not move the state
    # gradients flow only through valid steps
    x = packed.data.clone().requires_grad_(True)
    m.ForwardPacked(nn.PackedSequence(x, packed.lengths))[0].data.sum().backward()
    assert bool((x.grad[1, 2:] == 0).all()) and bool((x.grad[1, :2] != 0).any())
    assert [tuple(t.shape) for t in nn.UnpadSequence(padded, lengths)] == [(5, padded.shape[2]), (2, padded.shape[2]),
                                                                           (4, padded.shape[2])]


@pytest.mark.parametrize("kind", ["rnn", "lstm", "gru"])
def test_stacks_match_torch_stacks(kind):
    torch.manual_seed(0)
    ours = {"rnn": nn.RNN, "lstm": nn.LSTM, "gru": nn.GRU}[kind](3, 5, num_layers=2, bidirectional=True, dtype=D)
    ref = {"rnn": torch.nn.RNN, "lstm": torch.nn.LSTM, "gru": torch.nn.GRU}[kind](
        3, 5, num_layers=2, bidirectional=True, batch_first=True).double()
    with torch.no_grad():
        for l in range(2):
            for d, cells in enumerate((ours.cells, ours.backcells)):
                suf = f"_l{l}" + ("_reverse" if d else "")
                getattr(ref, "weight_ih" + suf).copy_(cells[l].wih.weight)
                getattr(ref, "weight_hh" + suf).copy_(cells[l].whh.weight)
                getattr(ref, "bias_ih" + suf).copy_(cells[l].wih.bias)
                bhh = cells[l].whh.bias
                getattr(ref, "bias_hh" + suf).copy_(bhh if bhh is not None else torch.zeros(ref.hidden_size * {"rnn": 1, "lstm": 4, "gru": 3}[kind], dtype=D))
    x = _x(2, 6, 3)
    out, st = ours.ForwardWithState(x)
    rout, rst = ref(x)
    assert torch.allclose(out, rout, rtol=1e-10, atol=1e-12)
    h, rh = (st[0], rst[0]) if kind == "lstm" else (st, rst)
    assert torch.allclose(h, rh, rtol=1e-10, atol=1e-12)


@pytest.mark.parametrize("kw", [dict(stride=2, padding=1), dict(dilation=2, padding=2), dict(groups=2),
                                dict(groups=4, stride=(2, 1), padding=(0, 2)),
                                dict(padding=1, padding_mode="reflect"), dict(padding=2, padding_mode="circular"),
                                dict(padding=1, padding_mode="replicate"), dict(bias=False)])
def test_conv2d_options_match_torch(kw):
    torch.manual_seed(0)
    ours = nn.Conv2d(4, 8, 3, dtype=D, **kw)
    ref = torch.nn.Conv2d(4, 8, 3, **kw).double()
    with torch.no_grad():
        ref.weight.copy_(ours.weight)
        if ours.bias is not None:
            ref.bias.copy_(ours.bias)
    x = _x(2, 4, 9, 8).requires_grad_(True)
    xr = x.detach().clone().requires_grad_(True)
    y, yr = ours(x), ref(xr)
    assert y.shape == yr.shape and torch.allclose(y, yr, rtol=1e-10, atol=1e-12)
    g = _x(*y.shape, seed=5)
    y.backward(g)
    yr.backward(g)
    assert torch.allclose(x.grad, xr.grad, rtol=1e-9, atol=1e-12)
    assert torch.allclose(ours.weight.grad, ref.weight.grad, rtol=1e-9, atol=1e-11)


def test_conv1d_3d_transpose_options_match_torch():
    torch.manual_seed(0)
    for ours, ref, shape in (
            (nn.Conv1d(4, 6, 3, stride=2, padding=1, dilation=2, groups=2, dtype=D),
             torch.nn.Conv1d(4, 6, 3, stride=2, padding=1, dilation=2, groups=2), (2, 4, 11)),
            (nn.Conv3d(2, 4, (2, 3, 2), stride=(1, 2, 1), padding=(1, 0, 1), dtype=D),
             torch.nn.Conv3d(2, 4, (2, 3, 2), stride=(1, 2, 1), padding=(1, 0, 1)), (1, 2, 4, 7, 5)),
            (nn.ConvTranspose2d(4, 6, 3, stride=2, padding=1, output_padding=1, dtype=D),
             torch.nn.ConvTranspose2d(4, 6, 3, stride=2, padding=1, output_padding=1), (2, 4, 5, 4)),
            (nn.ConvTranspose1d(4, 4, 4, stride=3, groups=2, dtype=D),
             torch.nn.ConvTranspose1d(4, 4, 4, stride=3, groups=2), (2, 4, 6)),
            (nn.ConvTranspose3d(2, 3, 2, stride=2, dtype=D), torch.nn.ConvTranspose3d(2, 3, 2, stride=2), (1, 2, 3, 3, 2))):
        ref = ref.double()
        with torch.no_grad():
            ref.weight.copy_(ours.weight)
            ref.bias.copy_(ours.bias)
        x = _x(*shape)
        assert torch.allclose(ours(x), ref(x), rtol=1e-10, atol=1e-12), type(ours).__name__


def test_pool_options_match_torch():
    x = _x(2, 3, 9, 10)
    cases = [
        (nn.MaxPool2d(3, 2, 1), lambda t: F.max_pool2d(t, 3, 2, 1)),
        (nn.MaxPool2d(2, 2, 0, dilation=2), lambda t: F.max_pool2d(t, 2, 2, 0, dilation=2)),
        (nn.MaxPool2d(3, 2, 0, ceil_mode=True), lambda t: F.max_pool2d(t, 3, 2, 0, ceil_mode=True)),
        (nn.AvgPool2d(3, 2, 1), lambda t: F.avg_pool2d(t, 3, 2, 1)),
        (nn.AvgPool2d(3, 2, 1, count_include_pad=False), lambda t: F.avg_pool2d(t, 3, 2, 1, count_include_pad=False)),
        (nn.AvgPool2d(2, 2, 0, ceil_mode=True), lambda t: F.avg_pool2d(t, 2, 2, 0, ceil_mode=True)),
    ]
    for ours, ref in cases:
        assert torch.allclose(ours(x), ref(x), rtol=1e-12, atol=1e-14), ours
    x1, x3 = _x(2, 3, 11), _x(1, 2, 5, 6, 4)
    assert torch.equal(nn.MaxPool1d(3, 2, 1)(x1), F.max_pool1d(x1, 3, 2, 1))
    assert torch.allclose(nn.AvgPool3d(2)(x3), F.avg_pool3d(x3, 2), rtol=1e-12)
    assert torch.equal(nn.MaxPool3d(2, 1)(x3), F.max_pool3d(x3, 2, 1))


def test_concurrent_backward_into_shared_leaves_is_exact():
    """Several threads each build a graph over the same parameters and run backward; with
    integer-valued gradients the accumulated sum is exact in any order."""
    lin = nn.Linear(6, 4, dtype=D)
    with torch.no_grad():
        lin.weight.copy_(torch.randint(-3, 4, (4, 6)).to(D))
        lin.bias.zero_()
    xs = [torch.randint(-2, 3, (5, 6), generator=torch.Generator().manual_seed(i)).to(D) for i in range(8)]
    want_w = sum(torch.ones(5, 4, dtype=D).t() @ x for x in xs)
    errs = []

    def work(x):
        try:
            lin(x).sum().backward()
        except Exception as e:          # noqa: BLE001
            errs.append(e)

    for _ in range(3):
        lin.zero_grad()
        ts = [threading.Thread(target=work, args=(x,)) for x in xs]
        [t.start() for t in ts]
        [t.join() for t in ts]
        assert not errs
        assert torch.equal(lin.weight.grad, want_w) and torch.equal(lin.bias.grad, torch.full((4,), 40.0, dtype=D))


def test_index_maps_are_range_checked_before_upload():
    import numpy as np
    from gonn_b200.ops.window import device_maps
    good = np.array([[0, 1, -1], [2, 3, 3]], dtype=np.int32)
    assert device_maps(good, 4, "cpu", True)["idx"].shape == (2, 3)
    with pytest.raises(ValueError):
        device_maps(np.array([[0, 4]], dtype=np.int32), 4, "cpu", False)
    with pytest.raises(ValueError):
        device_maps(np.array([[-2, 1]], dtype=np.int32), 4, "cpu", False)


def test_attention_layer_trains_with_adam():
    """Thirty Adam steps on a fixed regression target through MultiHeadAttention: the loss must
    fall by a large factor (the reference's benchmark/flashbwd/main.go:97-121 check)."""
    from gonn_b200 import optim
    torch.manual_seed(0)
    mha = nn.MultiHeadAttention(16, 2, dtype=D)
    x, target = _x(4, 6, 16, seed=1), _x(4, 6, 16, seed=2) * 0.1
    opt = optim.Adam(mha.parameters(), lr=0.02)
    losses = []
    for _ in range(30):
        opt.zero_grad()
        loss = nn.MSELoss(mha(x, x, x, True), target)
        loss.backward()
        opt.step()
        losses.append(float(loss))
    assert losses[-1] < 0.25 * losses[0], losses[::10]

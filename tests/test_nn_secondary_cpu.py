"""Secondary nn components against closed forms or the PyTorch layer of the same name
(CPU, float64).  One test per behaviour of the reference's smaller layers."""
import math

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from gonn_b200 import nn

D = torch.float64


def _x(*shape, seed=0):
    return torch.randn(*shape, dtype=D, generator=torch.Generator().manual_seed(seed))


def test_max_unpool_round_trip_and_sizes():
    x = _x(2, 3, 6, 8)
    pool = nn.MaxPool2d(2)
    y, idx = pool.ForwardWithIndices(x)
    ty, tidx = F.max_pool2d(x, 2, return_indices=True)
    assert torch.equal(y, ty) and torch.equal(idx.long(), tidx)
    up = nn.MaxUnpool2d(2)(y, idx)
    assert torch.equal(up, F.max_unpool2d(ty, tidx, 2))
    # default size (in-1)*stride + kernel; explicit size; range check
    y1, i1 = nn.MaxPool1d(3, 2).ForwardWithIndices(_x(1, 1, 9))
    assert nn.MaxUnpool1d(3, 2)(y1, i1).shape == (1, 1, (4 - 1) * 2 + 3)
    assert nn.MaxUnpool1d(3, 2)(y1, i1, output_size=(10,)).shape == (1, 1, 10)
    with pytest.raises(ValueError):
        nn.MaxUnpool1d(3, 2)(y1, i1, output_size=(3,))
    # gradient gathers at the same indices
    yy = y.clone().requires_grad_(True)
    nn.MaxUnpool2d(2)(yy, idx).pow(2).sum().backward()
    assert torch.allclose(yy.grad, 2 * y)


def test_pixel_and_channel_shuffle():
    x = _x(2, 8, 3, 5)
    assert torch.equal(nn.PixelShuffle(2)(x), F.pixel_shuffle(x, 2))
    z = _x(2, 2, 6, 4)
    assert torch.equal(nn.PixelUnshuffle(2)(z), F.pixel_unshuffle(z, 2))
    assert torch.equal(nn.PixelUnshuffle(2)(nn.PixelShuffle(2)(x)), x)
    assert torch.equal(nn.ChannelShuffle(4)(x), F.channel_shuffle(x, 4))


def test_cosine_similarity_adds_eps_to_the_product():
    a, b = _x(5, 7), _x(5, 7, seed=1)
    want = (a * b).sum(1) / (a.norm(dim=1) * b.norm(dim=1) + 1e-8)
    assert torch.allclose(nn.CosineSimilarity()(a, b), want, rtol=1e-13, atol=0)
    z = torch.zeros(2, 3, dtype=D)
    assert torch.equal(nn.CosineSimilarity()(z, z), torch.zeros(2, dtype=D))   # 0 / eps, not NaN


def test_pairwise_distance():
    a, b = _x(4, 6), _x(4, 6, seed=2)
    for p in (1.0, 2.0, 3.0):
        want = ((a - b + 1e-6).abs() ** p).sum(-1) ** (1 / p)
        assert torch.allclose(nn.PairwiseDistance(p)(a, b), want, rtol=1e-13)
    assert torch.allclose(nn.PairwiseDistance()(a, b), F.pairwise_distance(a, b), rtol=1e-12)


def test_local_response_norm_window_and_divisor():
    x = _x(2, 7, 3, 2)
    for n in (3, 4, 5):
        got = nn.LocalResponseNorm(n, alpha=1e-2, beta=0.6, k=1.5)(x)
        assert torch.allclose(got, F.local_response_norm(x, n, 1e-2, 0.6, 1.5), rtol=1e-12), n
    # written out: window [c - n/2, c + (n-1)/2] clamped, divisor always n
    n, C = 4, 7
    sq = x ** 2
    want = torch.empty_like(x)
    for c in range(C):
        lo, hi = max(c - n // 2, 0), min(c + (n - 1) // 2, C - 1)
        want[:, c] = x[:, c] / (1.0 + 1e-4 / n * sq[:, lo:hi + 1].sum(1)) ** 0.75
    assert torch.allclose(nn.LocalResponseNorm(4)(x), want, rtol=1e-12)


def test_upsample_modes_match_torch():
    x = _x(2, 3, 4, 5)
    for mode, ac in (("nearest", False), ("bilinear", False), ("bilinear", True), ("bicubic", False), ("bicubic", True)):
        kw = {} if mode == "nearest" else {"align_corners": ac}
        want = F.interpolate(x, scale_factor=2, mode=mode, **kw)
        got = nn.Upsample(2, mode, ac)(x)
        assert got.shape == want.shape and torch.allclose(got, want, rtol=1e-10, atol=1e-12), (mode, ac)
    x1 = _x(2, 3, 6)
    assert torch.allclose(nn.Upsample(3, "linear")(x1), F.interpolate(x1, scale_factor=3, mode="linear"), rtol=1e-12)


def test_fractional_max_pool_window_starts():
    x = _x(1, 2, 9, 11)
    k, out, u = (2, 3), (4, 5), [0.3, 0.8]
    got = nn.FractionalMaxPool2d(k, out, samples=u)(x)
    starts = []
    for d, n_in in enumerate((9, 11)):
        alpha = (n_in - k[d]) / (out[d] - 1)
        st = [math.floor((i + u[d]) * alpha) - math.floor(u[d] * alpha) for i in range(out[d])]
        st[-1] = n_in - k[d]
        starts.append(st)
    want = torch.stack([torch.stack([x[:, :, a:a + k[0], b:b + k[1]].amax((-1, -2)) for b in starts[1]], -1)
                        for a in starts[0]], -2)
    assert torch.equal(got, want)
    assert nn.FractionalMaxPool2d(2, (4, 5))(x).shape == (1, 2, 4, 5)          # random u per call
    with pytest.raises(ValueError):
        nn.FractionalMaxPool2d(6, (5, 5))(x)                                    # k + out - 1 > in
    assert nn.FractionalMaxPool3d(2, 2, samples=[0.5, 0.5, 0.5])(_x(1, 1, 4, 4, 4)).shape == (1, 1, 2, 2, 2)


def test_lp_pool_is_a_sum_not_a_mean():
    x = _x(2, 3, 6, 6).abs()
    for p in (1.0, 2.0, 3.0):
        assert torch.allclose(nn.LPPool2d(p, 2)(x), F.lp_pool2d(x, p, 2), rtol=1e-12)
    assert torch.allclose(nn.LPPool1d(2.0, 3, 2)(x[:, :, 0]), F.lp_pool1d(x[:, :, 0], 2.0, 3, 2), rtol=1e-12)
    w = x[:, :, :2, :2]
    assert torch.allclose(nn.LPPool2d(2.0, 2)(x)[:, :, 0, 0], (w ** 2).sum((-1, -2)).sqrt(), rtol=1e-12)


def test_adaptive_pool_windows():
    x = _x(2, 3, 7, 10)
    for out in ((3, 4), (7, 10), (1, 1), (5, 3)):
        assert torch.allclose(nn.AdaptiveAvgPool2d(out)(x), F.adaptive_avg_pool2d(x, out), rtol=1e-12), out
        assert torch.equal(nn.AdaptiveMaxPool2d(out)(x), F.adaptive_max_pool2d(x, out)), out
    x1 = _x(2, 3, 11)
    assert torch.allclose(nn.AdaptiveAvgPool1d(4)(x1), F.adaptive_avg_pool1d(x1, 4), rtol=1e-12)
    x3 = _x(1, 2, 5, 6, 7)
    assert torch.equal(nn.AdaptiveMaxPool3d((2, 3, 4))(x3), F.adaptive_max_pool3d(x3, (2, 3, 4)))


def test_channel_dropout_masks_whole_channels():
    torch.manual_seed(0)
    x = torch.ones(8, 16, 5, 5, dtype=D)
    m = nn.Dropout2d(0.25)
    y = m(x)
    per = y.reshape(8, 16, -1)
    assert bool(((per == 0).all(-1) | (per == 1 / 0.75).all(-1)).all())        # all-or-nothing, scaled 1/(1-p)
    assert 0 < int((per[:, :, 0] == 0).sum()) < 8 * 16
    m.eval()
    assert torch.equal(m(x), x)
    with pytest.raises(ValueError):
        nn.Dropout2d(0.5).train()(torch.ones(3, dtype=D))
    assert nn.Dropout1d(0.5)(torch.ones(4, 6, 9, dtype=D)).shape == (4, 6, 9)
    assert nn.Dropout3d(0.5)(torch.ones(2, 3, 2, 2, 2, dtype=D)).shape == (2, 3, 2, 2, 2)


def test_alpha_dropout_constants_and_moments():
    torch.manual_seed(1)
    p = 0.2
    q = 1 - p
    ap = -1.7580993408473766
    a = (q + ap * ap * q * (1 - q)) ** -0.5
    b = -a * ap * (1 - q)
    x = _x(200, 500)
    y = nn.AlphaDropout(p)(x)
    kept = torch.isclose(y, a * x + b, rtol=1e-12, atol=1e-12)
    dropped = torch.isclose(y, torch.full_like(y, a * ap + b), rtol=1e-12, atol=1e-12)
    assert bool((kept | dropped).all()) and abs(float(dropped.double().mean()) - p) < 0.01
    assert abs(float(y.mean())) < 0.02 and abs(float(y.std()) - 1) < 0.02     # self-normalising
    f = nn.FeatureAlphaDropout(0.5)(torch.ones(4, 32, 6, dtype=D))
    assert bool((f == f[:, :, :1]).all())                                      # one decision per channel
    e = nn.AlphaDropout(0.5).eval()
    assert torch.equal(e(x), x)


def test_weight_norm_wrappers():
    torch.manual_seed(0)
    lin = nn.Linear(5, 4, dtype=D)
    w0, x = lin.weight.detach().clone(), _x(3, 5)
    wn = nn.WeightNormLinear(lin)
    assert sorted(n for n, _ in wn.named_parameters()) == ["bias", "weight_g", "weight_v"]
    assert torch.allclose(wn.weight_g.reshape(-1), w0.norm(dim=1)) and torch.allclose(wn(x), lin(x), rtol=1e-12)
    with torch.no_grad():
        wn.weight_g.mul_(2.0)                               # direction unchanged, length doubled
    assert torch.allclose(wn.EffectiveWeight(), 2 * w0, rtol=1e-12)
    baked = nn.RemoveWeightNormLinear(wn)
    assert isinstance(baked, nn.Linear) and torch.allclose(baked.weight, 2 * w0, rtol=1e-12)
    assert torch.allclose(baked(x), wn(x), rtol=1e-12)
    conv = nn.Conv2d(2, 3, 3, dtype=D)
    wc = nn.WeightNormConv2d(conv)
    img = _x(1, 2, 5, 5)
    assert wc.weight_g.numel() == 3 and torch.allclose(wc(img), conv(img), rtol=1e-12)
    wc(img).sum().backward()
    assert wc.weight_g.grad is not None and wc.weight_v.grad is not None
    assert torch.allclose(nn.RemoveWeightNormConv2d(wc)(img), conv(img), rtol=1e-12)


def test_spectral_norm_wrappers():
    torch.manual_seed(0)
    lin = nn.Linear(6, 4, dtype=D)
    sn = nn.SpectralNormLinear(lin)
    assert sn.weight_orig is lin.weight and sorted(n for n, _ in sn.named_buffers()) == ["u", "v"]
    assert sorted(n for n, _ in sn.named_parameters()) == ["bias", "weight_orig"]
    for _ in range(30):                                     # training forwards refine u, v
        sn(_x(2, 6))
    true_sigma = float(torch.linalg.svdvals(lin.weight.detach())[0])
    assert abs(sn.EstimatedSigma() - true_sigma) < 1e-6 * true_sigma
    assert abs(float(torch.linalg.svdvals(sn.EffectiveWeight().detach())[0]) - 1.0) < 1e-6
    sn.eval()
    u0 = sn.u.clone()
    sn(_x(2, 6))
    assert torch.equal(sn.u, u0)                            # no power iteration in eval
    # sigma = u^T W v is differentiable with respect to W with u, v held constant
    sn.EffectiveWeight().sum().backward()
    W, u, v = lin.weight.detach(), sn.u, sn.v
    sigma = u @ W @ v
    want = torch.ones_like(W) / sigma - W.sum() / sigma ** 2 * torch.outer(u, v)
    assert torch.allclose(lin.weight.grad, want, rtol=1e-9, atol=1e-12)
    baked = nn.RemoveSpectralNormLinear(sn)
    assert torch.allclose(baked.weight, W / sigma, rtol=1e-12)
    sc = nn.SpectralNormConv2d(nn.Conv2d(2, 3, 3, dtype=D), n_power_iterations=2)
    assert sc.u.numel() == 3 and sc.v.numel() == 2 * 9 and sc(_x(1, 2, 5, 5)).shape == (1, 3, 3, 3)


def test_generic_parametrizations():
    torch.manual_seed(0)
    lin = nn.Linear(4, 4, dtype=D)
    w0 = lin.weight.detach().clone()
    pl = nn.ParametrizedLinear(lin, nn.ParametrizationFunc(lambda w: (w + w.t()) / 2))
    assert "weight_orig" in dict(pl.named_parameters()) and nn.IsParametrized(pl) and not nn.IsParametrized(lin)
    assert torch.allclose(pl.EffectiveWeight(), (w0 + w0.t()) / 2)
    pl.AddParametrization(nn.ParametrizationFunc(lambda w: 2 * w))          # applied in registration order
    assert torch.allclose(pl.EffectiveWeight(), w0 + w0.t())
    with pytest.raises(Exception):
        pl.AddParametrization(nn.ParametrizationFunc(lambda w: w[:2]))      # must preserve the shape
    with pytest.raises(ValueError):
        pl.SetEffectiveWeight(torch.eye(4, dtype=D))                        # chain has no right inverse
    inv = nn.ParametrizedLinear(nn.Linear(3, 3, dtype=D), nn.InvertibleParametrization(torch.exp, torch.log))
    target = torch.full((3, 3), 2.0, dtype=D)
    inv.SetEffectiveWeight(target)
    assert torch.allclose(inv.EffectiveWeight(), target, rtol=1e-12)
    assert torch.allclose(inv.weight_orig, target.log(), rtol=1e-12)
    calls = []
    cnt = nn.ParametrizedLinear(nn.Linear(3, 2, dtype=D), nn.ParametrizationFunc(lambda w: calls.append(1) or w * 1.0))
    x = _x(2, 3)
    cnt(x), cnt(x)
    n_plain = len(calls)
    with cnt.Cached():
        a, b = cnt(x), cnt(x)
        (a + b).sum().backward()
    assert len(calls) == n_plain + 1 and cnt.weight_orig.grad is not None   # evaluated once inside the window
    plain = nn.RemoveParametrizations(pl)
    assert isinstance(plain, nn.Linear) and torch.allclose(plain.weight, w0 + w0.t())


def test_prune_registry():
    from gonn_b200.nn import prune
    torch.manual_seed(0)
    lin = nn.Linear(6, 5, dtype=D)
    w = lin.weight
    w0 = w.detach().clone()
    prune.L1Unstructured(w, 0.4)
    k = round(0.4 * 30)
    assert prune.IsPruned(w) and int((w == 0).sum()) == k
    thresh = w0.abs().flatten().sort().values[k - 1]
    assert bool((w0.abs()[w == 0] <= thresh).all()) and torch.equal(prune.Orig(w), w0)
    prune.L1Unstructured(w, 0.5)        # k = round(amount * n) of ALL entries, zeros sort first: 15 in total
    assert int((w == 0).sum()) == 15 and torch.equal(prune.Orig(w), w0)
    with torch.no_grad():
        w.add_(1.0)                                           # an optimizer step revives pruned entries
    prune.Reapply(w)
    assert int((w == 0).sum()) == 15
    prune.Remove(w)
    assert not prune.IsPruned(w)
    v = nn.Linear(6, 5, dtype=D).weight
    prune.LnStructured(v, 0.4, 2, 0)                          # two of five rows, smallest L2 norm
    zero_rows = (v == 0).all(1)
    assert int(zero_rows.sum()) == 2
    r1, r2 = nn.Linear(6, 5, dtype=D).weight, nn.Linear(6, 5, dtype=D).weight
    with torch.no_grad():
        r2.copy_(r1)
    prune.RandomUnstructured(r1, 0.3, seed=5)
    prune.RandomUnstructured(r2, 0.3, seed=5)
    assert torch.equal(r1, r2) and int((r1 == 0).sum()) == 9
    a, b = nn.Linear(4, 4, dtype=D).weight, nn.Linear(4, 4, dtype=D).weight
    with torch.no_grad():
        a.copy_(a.sign() * (a.abs() + 10.0))               # every entry of a outweighs every entry of b
    prune.GlobalUnstructured([a, b], 0.5)
    assert int((a == 0).sum()) == 0 and int((b == 0).sum()) == 16
    m = torch.zeros(4, 4, dtype=D)
    m[0] = 1
    c = nn.Linear(4, 4, dtype=D).weight
    prune.CustomFromMask(c, m)
    assert torch.equal(prune.Mask(c), m) and bool((c[1:] == 0).all())


def test_lazy_modules_materialise_on_first_forward():
    torch.manual_seed(0)
    m = nn.LazyLinear(7)
    assert nn.IsLazy(m) and len(list(m.parameters())) == 0
    m.eval()
    y = m(torch.randn(3, 5))
    assert y.shape == (3, 7) and not nn.IsLazy(m) and not m.inner.training
    assert sorted(n for n, _ in m.named_parameters()) == ["inner.bias", "inner.weight"]
    assert tuple(m.inner.weight.shape) == (7, 5)
    c = nn.LazyConv2d(4, 3, padding=1)
    assert c(torch.randn(2, 6, 5, 5)).shape == (2, 4, 5, 5) and c.inner.weight.shape[1] == 6
    b = nn.LazyBatchNorm1d()
    assert b(torch.randn(4, 9)).shape == (4, 9) and b.inner.weight.numel() == 9


def test_embedding_bag_modes():
    torch.manual_seed(0)
    idx = torch.tensor([1, 2, 4, 5, 4, 3, 2, 9])
    off = torch.tensor([0, 4, 4])                             # the middle bag is empty
    for mode in ("sum", "mean", "max"):
        eb = nn.EmbeddingBag(10, 3, mode, dtype=D)
        got = eb(idx, off)
        want = F.embedding_bag(idx, eb.weight, off, mode=mode)
        assert torch.allclose(got, want, rtol=1e-12), mode
        assert torch.equal(got[1], torch.zeros(3, dtype=D))
        got.sum().backward()
        assert eb.weight.grad is not None
    pad = nn.EmbeddingBag(10, 3, "mean", padding_idx=2, dtype=D)
    got = pad(idx, off)
    assert torch.allclose(got, F.embedding_bag(idx, pad.weight, off, mode="mean", padding_idx=2), rtol=1e-12)
    assert torch.allclose(pad(torch.tensor([[1, 2], [2, 2]]))[1], torch.zeros(3, dtype=D))   # all padding
    with pytest.raises(ValueError):
        pad(idx, torch.tensor([1, 3]))


def test_adaptive_log_softmax_with_loss():
    torch.manual_seed(0)
    m = nn.AdaptiveLogSoftmaxWithLoss(16, 20, [4, 10], div_value=2.0, dtype=D)
    names = [n for n, _ in m.named_parameters()]
    assert names == ["head.weight", "tail.0.0.weight", "tail.0.1.weight", "tail.1.0.weight", "tail.1.1.weight"]
    assert tuple(m.head.weight.shape) == (4 + 2, 16)
    assert tuple(m.tail[0][0].weight.shape) == (8, 16) and tuple(m.tail[0][1].weight.shape) == (6, 8)
    assert tuple(m.tail[1][0].weight.shape) == (4, 16) and tuple(m.tail[1][1].weight.shape) == (10, 4)
    x = _x(7, 16)
    lp = m.LogProb(x)
    assert lp.shape == (7, 20) and torch.allclose(lp.exp().sum(1), torch.ones(7, dtype=D), rtol=1e-12)
    t = torch.tensor([0, 3, 4, 9, 10, 19, 5])
    out, loss = m(x, t)
    assert torch.allclose(out, lp[torch.arange(7), t], rtol=1e-12) and torch.allclose(loss, -out.mean())
    assert torch.equal(m.Predict(x), lp.argmax(1))
    ref = torch.nn.AdaptiveLogSoftmaxWithLoss(16, 20, [4, 10], div_value=2.0).double()
    with torch.no_grad():
        ref.head.weight.copy_(m.head.weight)
        for i in range(2):
            ref.tail[i][0].weight.copy_(m.tail[i][0].weight)
            ref.tail[i][1].weight.copy_(m.tail[i][1].weight)
    assert torch.allclose(ref.log_prob(x), lp, rtol=1e-10)


def test_ctc_loss_matches_torch_and_handles_infeasible():
    torch.manual_seed(0)
    T, N, C, S = 12, 3, 6, 4
    lp = torch.randn(T, N, C, dtype=D).log_softmax(-1).requires_grad_(True)
    tg = torch.tensor([[1, 2, 2, 3], [4, 1, 5, 0], [2, 0, 0, 0]])
    il, tl = torch.tensor([12, 10, 7]), torch.tensor([4, 3, 1])
    for red in ("mean", "sum", "none"):
        got = nn.CTCLoss(lp, tg, il, tl, reduction=red)
        want = F.ctc_loss(lp, tg, il, tl, blank=0, reduction=red)
        assert torch.allclose(got, want, rtol=1e-10), red
    # gradient with respect to the logits (torch's kernel folds the log-softmax Jacobian into its
    # backward, so the two are comparable there, not at log_probs)
    z = torch.randn(T, N, C, dtype=D, requires_grad=True)
    g1, = torch.autograd.grad(nn.CTCLoss(z.log_softmax(-1), tg, il, tl), z)
    g2, = torch.autograd.grad(F.ctc_loss(z.log_softmax(-1), tg, il, tl), z)
    assert torch.allclose(g1, g2, rtol=1e-8, atol=1e-12)
    # at log_probs the gradient is -exp(alpha + beta - lp + loss): never positive, zero past the input length
    g, = torch.autograd.grad(nn.CTCLoss(lp, tg, il, tl, reduction="sum"), lp)
    assert bool((g <= 0).all()) and bool((g[7:, 2] == 0).all()) and bool((g[:7, 2].sum(-1) < 0).all())
    # a repeated label needs a blank in between: 3 frames cannot emit "1 1"
    short = torch.randn(3, 1, C, dtype=D).log_softmax(-1).requires_grad_(True)
    loss = nn.CTCLoss(short, torch.tensor([[1, 1]]), torch.tensor([2]), torch.tensor([2]), reduction="sum")
    assert math.isinf(float(loss))
    g, = torch.autograd.grad(loss, short)
    assert torch.equal(g, torch.zeros_like(g))

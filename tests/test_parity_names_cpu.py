"""Names and call forms of the reference that have no PyTorch spelling: constructor functions,
small record types, argument orders of the padding layers, transform objects."""
import math

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from gonn_b200 import backend, data, ml, nn, optim, quant
from gonn_b200 import tensor as T


def test_padding_argument_orders_follow_the_reference():
    x = torch.arange(2 * 2 * 3 * 4 * 5, dtype=torch.float64).reshape(2, 2, 3, 4, 5)
    p3 = (1, 2, 0, 1, 2, 1)                                  # left, right, top, bottom, front, back
    for cls, mode in ((nn.ZeroPad3d, "constant"), (nn.ReflectionPad3d, "reflect"),
                      (nn.ReplicationPad3d, "replicate"), (nn.CircularPad3d, "circular")):
        assert torch.equal(cls(*p3)(x), F.pad(x, p3, mode=mode)), cls.__name__
        assert torch.equal(cls(p3)(x), F.pad(x, p3, mode=mode))
    assert torch.equal(nn.ConstantPad3d(*p3, 7.5)(x), F.pad(x, p3, value=7.5))
    x2 = x[0]
    # the 2-D zero / constant / reflection / replication layers: top, bottom, left, right
    assert torch.equal(nn.ZeroPad2d(1, 2, 3, 0)(x2), F.pad(x2, (3, 0, 1, 2)))
    assert torch.equal(nn.ConstantPad2d(1, 2, 3, 0, -1.0)(x2), F.pad(x2, (3, 0, 1, 2), value=-1.0))
    assert torch.equal(nn.ConstantPad2d((1, 2, 3, 0), -1.0)(x2), F.pad(x2, (3, 0, 1, 2), value=-1.0))
    assert torch.equal(nn.ReplicationPad2d(1, 2, 3, 0)(x2), F.pad(x2, (3, 0, 1, 2), mode="replicate"))
    assert torch.equal(nn.ReflectionPad2d(1)(x2), F.pad(x2, (1, 1, 1, 1), mode="reflect"))
    # CircularPad2d alone takes PyTorch's order
    assert torch.equal(nn.CircularPad2d(1, 2, 3, 0)(x2), F.pad(x2, (1, 2, 3, 0), mode="circular"))
    x1 = x2[0]
    assert torch.equal(nn.ZeroPad1d(2, 1)(x1), F.pad(x1, (2, 1)))
    assert torch.equal(nn.ConstantPad1d(2, 1, 9.0)(x1), F.pad(x1, (2, 1), value=9.0))
    assert torch.equal(nn.ConstantPad1d(2, 9.0)(x1), F.pad(x1, (2, 2), value=9.0))
    with pytest.raises(ValueError):
        nn.ZeroPad3d(1, 2, 3)


def test_constructor_aliases_and_small_types():
    lin = nn.NewLinear(3, 4)
    assert isinstance(lin, nn.Linear) and nn.NewLSTM.__wrapped__ is nn.LSTM and nn.NewZeroPad1d.__wrapped__ is nn.ZeroPad1d
    assert isinstance(nn.NewLazyLinear(5), torch.nn.Module)
    ln = nn.NewLayerNormShape([3, 4])
    assert tuple(ln.weight.shape) == (3, 4)
    assert optim.NewAdam.__wrapped__ is optim.Adam and optim.NewStepLR.__wrapped__ is optim.StepLR
    assert data.NewTensorDataset.__wrapped__ is data.TensorDataset and data.NewDataLoader.__wrapped__ is data.DataLoader
    assert isinstance(lin, nn.Child) and nn.Base is nn.Module
    assert isinstance(nn.ParametrizedLinear, type)
    p = nn.Param("weight", lin.weight)
    assert p.Name == "weight" and p.T is lin.weight
    assert nn.ReduceSum == "sum" and nn.Reduction.ReduceNone == "none"
    a, b = torch.randn(4, 3), torch.randn(4, 3)
    assert torch.equal(nn.MSELoss(a, b, reduction=nn.ReduceSum), nn.MSELoss(a, b, reduction="sum"))
    assert nn.MSELoss(a, b, reduction=nn.ReduceNone).shape == (4, 3)
    assert issubclass(backend.NativeBackend, backend.Elementwiser)
    assert backend.Elementwiser().Unary(backend.UnaryKind.ReLU, a) is None


def test_lstm_state_record_and_seeded_rrelu():
    cell = nn.LSTMCell(3, 5, dtype=torch.float64)
    x = torch.randn(2, 3, dtype=torch.float64)
    st = nn.LSTMState(torch.zeros(2, 5, dtype=torch.float64), torch.zeros(2, 5, dtype=torch.float64))
    h1, c1 = cell(x, st)
    h2, c2 = cell(x)
    assert torch.equal(h1, h2) and torch.equal(c1, c2) and st.H is st[0]
    x = torch.randn(64, dtype=torch.float64)
    r = nn.RReLULayer(0.1, 0.3, per_element=False)
    y1, y2 = r.Seed(7)(x), r.Seed(7)(x)
    assert torch.equal(y1, y2)
    neg = x < 0
    slope = (y1[neg] / x[neg])
    assert torch.allclose(slope, slope[0].expand_as(slope)) and 0.1 <= float(slope[0]) <= 0.3
    e = nn.RReLU(0.1, 0.3).Seed(3)
    z1 = e(x)
    z2 = nn.RReLU(0.1, 0.3).Seed(3)(x)
    assert torch.equal(z1, z2) and (z1[neg] / x[neg]).min() >= 0.1 - 1e-12
    r.eval()
    assert torch.allclose(r(x)[neg], x[neg] * 0.2)


def test_tensor_type_names_and_printing():
    assert T.DType is torch.dtype and T.UnaryKind is backend.UnaryKind and T.UnaryGELUExact == 7
    assert T.String(torch.tensor([1.0, 2.5], dtype=torch.float64)) == "Tensor(shape=[2], data=[1 2.5])"
    s = T.String(torch.arange(20, dtype=torch.float32).requires_grad_(True))
    assert s == ("Tensor(shape=[20], data=[[0 1 2 3 4 5 6 7] ... [12 13 14 15 16 17 18 19]], dtype=float32, "
                 "requires_grad=true)")
    x = torch.tensor([1.0, 2.0], requires_grad=True)
    f = T.Function("square", [x], [2.0], lambda g, saved, ins: [g * saved[0] * ins[0]])
    f.Apply(lambda a: a * a).sum().backward()
    assert torch.equal(x.grad, torch.tensor([2.0, 4.0]))
    with pytest.raises(Exception):
        T.Function("nograd", [x]).Apply(lambda a: a)


def test_transforms_are_objects_with_apply():
    img = torch.arange(2 * 4 * 6, dtype=torch.float64).reshape(2, 4, 6)
    n = data.Normalize([1.0, 2.0], [2.0, 4.0])
    assert isinstance(n, data.Transform) and torch.equal(n.Apply(img), n(img))
    assert torch.equal(n(img)[1], (img[1] - 2.0) / 4.0)
    with pytest.raises(ValueError):
        data.Normalize([0.0], [1.0]).Apply(img)
    with pytest.raises(ValueError):
        data.Normalize([0.0, 0.0], [1.0, 0.0]).Apply(img)
    assert torch.equal(data.RandomHorizontalFlip(1.0).Apply(img), img.flip(-1))
    assert torch.equal(data.RandomHorizontalFlip(0.0).Apply(img), img)
    c = data.RandomCrop([1, 2, 3], seed=0).Apply(img)
    assert c.shape == (1, 2, 3)
    assert data.RandomCrop(2, seed=1).Apply(img).shape == (2, 2, 2)
    assert data.RandomCrop([6], seed=1).Apply(img).shape == (2, 4, 6)
    with pytest.raises(ValueError):
        data.RandomCrop([5, 7]).Apply(img)
    assert data.ToFloat().Apply(img) is img
    assert data.ToFloat(1 / 255).Apply(torch.tensor([255], dtype=torch.uint8)).item() == pytest.approx(1.0)
    comp = data.Compose([data.RandomCrop([2, 2], seed=0), data.RandomHorizontalFlip(1.0)])
    assert comp.Apply(img).shape == (2, 2, 2) and len(comp.Transforms) == 2
    ds = data.TensorDataset(torch.randn(5, 2, 4, 6), torch.arange(5))
    batch = next(iter(data.DataLoader(ds, batch_size=2, transform=comp)))
    assert isinstance(batch, data.Batch) and batch.X.shape == (2, 2, 2, 2) and batch.Y.tolist() == [0, 1]
    xb, yb = batch
    assert xb is batch.X and yb is batch.Y


def test_quant_records_and_constructor_forms():
    w = torch.randn(6, 4, dtype=torch.float64)
    q = quant.Quantize(w)
    qc = quant.QuantizePerChannel(w, 0)
    assert q.Numel() == 24 and qc.Numel() == 24 and qc.Channels() == 6
    lin = nn.Linear(4, 6, dtype=torch.float64)
    x = torch.randn(3, 4, dtype=torch.float64)
    d = quant.NewDynamicLinearFrom(lin, quant.WithPerChannelWeights())
    assert torch.equal(d(x), quant.DynamicLinear(lin, per_channel_weights=True)(x))
    obs = quant.MinMaxObserver()
    obs.Observe(x)
    s = quant.NewStaticLinearFrom(lin, obs)
    assert (s.InScale, s.InZeroPoint) == tuple(obs.ComputeQParams())
    assert (s(x) - lin(x)).abs().max() < 0.1
    assert quant.NewFakeQuant(True).Symmetric and isinstance(quant.NewQATLinearFrom(lin), quant.QATLinear)


def test_cluster_labels_read_as_array_and_as_call():
    X = np.concatenate([np.random.default_rng(0).normal(0, 0.1, (20, 2)),
                        np.random.default_rng(1).normal(5, 0.1, (20, 2))])
    for m in (ml.KMeans(K=2, Seed=0), ml.DBSCAN(Eps=0.5, MinSamples=3), ml.AgglomerativeClustering(NClusters=2)):
        m.Fit(X)
        lab = m.Labels()
        assert type(lab) is np.ndarray and np.array_equal(lab, np.asarray(m.Labels)) and len(lab) == 40
        assert len(set(lab[:20])) == 1 and lab[0] != lab[-1], type(m).__name__


def test_method_spellings_on_tensors():
    from gonn_b200.tensor import methods
    assert len(methods.installed()) >= 90 and "T" not in methods.installed()
    x = T.SetRequiresGrad(T.New([1, -2, 3], 3))
    y = x.Add(T.Ones(3, dtype=torch.float64)).ReLU().Square().Sum()
    y.Backward()
    assert y.Item() == 20.0 and x.grad.tolist() == [4.0, 0.0, 8.0]
    assert x.Dim() == 1 and x.DType() == torch.float64 and x.Numel() == 3
    m = T.New([1, 2, 3, 4, 5, 6], 2, 3)
    assert m.Transpose().shape == (3, 2) and torch.equal(m.Transpose(), m.T)
    assert m.MatMul(m.Transpose()).tolist() == [[14.0, 32.0], [32.0, 77.0]]
    assert m.SumAxis(1, False).tolist() == [6.0, 15.0] and m.Reshape(3, 2).shape == (3, 2)
    assert m.Unary("square").Sum().Item() == 91.0 and m.String().startswith("Tensor(shape=[2 3]")
    assert torch.equal(m.Softmax(1).Sum().reshape(()), torch.tensor(2.0, dtype=torch.float64)) or \
        abs(m.Softmax(1).Sum().Item() - 2.0) < 1e-12
    # torch's own attributes are untouched
    assert torch.equal(m.T, m.t()) and m.sum().item() == 21.0


def test_forward_spelling_bypasses_hooks_like_the_reference():
    lin = nn.Linear(3, 2)
    x = torch.randn(4, 3)
    seen = []
    h = nn.RegisterForwardHook(lin, lambda m, inp, out: seen.append(1))
    assert torch.equal(lin.Forward(x), lin.forward(x)) and seen == []
    lin(x)
    assert seen == [1]
    assert nn.RemoveHook(h)
    mha = nn.MultiHeadAttention(8, 2)
    q = torch.randn(2, 5, 8)
    assert torch.equal(mha.Forward(q, q, q, True), mha(q, q, q, True))


def test_container_hook_and_loader_method_spellings():
    ml_ = nn.ModuleList([nn.Linear(2, 2), nn.ReLU()])
    assert ml_.Len() == 2 and ml_.Get(1) is ml_[1]
    md = nn.ModuleDict({"b": nn.ReLU(), "a": nn.Tanh()})
    assert md.Len() == 2 and md.Keys() == ["a", "b"]
    pl = nn.ParameterList([torch.zeros(2), torch.ones(3)])
    assert pl.Len() == 2 and pl.Get(1).shape == (3,)
    pd = nn.ParameterDict({"w": torch.zeros(2)})
    assert pd.Len() == 1
    lin = nn.Linear(3, 2)
    seen = []
    hid = lin.RegisterForwardHook(lambda m, x, y: seen.append("post"))
    pid = lin.RegisterForwardPreHook(lambda m, x: seen.append("pre"))
    bid = lin.RegisterFullBackwardHook(lambda m, g: seen.append("bwd"))
    lin(torch.randn(4, 3, requires_grad=True)).sum().backward()
    assert seen == ["pre", "post", "bwd"]
    assert lin.RemoveHook(hid) and lin.RemoveHook(pid) and lin.RemoveHook(bid) and not lin.RemoveHook(hid)
    lz = nn.LazyLinear(4)
    assert lz.Inner() is None
    lz(torch.randn(2, 3))
    assert isinstance(lz.Inner(), nn.Linear)
    dl = data.DataLoader(data.TensorDataset(torch.randn(10, 2), torch.arange(10)), batch_size=4)
    assert dl.Len() == 3 and data.DataLoader(dl.dataset, batch_size=4, drop_last=True).Len() == 2


def test_cluster_predict_and_probability_methods():
    rng = np.random.default_rng(0)
    X = np.concatenate([rng.normal(0, 0.2, (30, 2)), rng.normal(4, 0.2, (30, 2))])
    y = np.array([0] * 30 + [1] * 30)
    probe = np.array([[0.1, -0.1], [4.1, 3.9], [20.0, 20.0]])
    db = ml.DBSCAN(Eps=0.6, MinSamples=3).Fit(X)
    p = db.Predict(probe)
    assert p[0] == db.Labels()[0] and p[1] == db.Labels()[-1] and p[2] == -1       # too far: noise
    ag = ml.AgglomerativeClustering(NClusters=2).Fit(X)
    p = ag.Predict(probe)
    assert p[0] == ag.Labels()[0] and p[1] == ag.Labels()[-1] and p[2] == p[1]     # nearest training point
    ms = ml.MeanShift(Bandwidth=1.0).Fit(X)
    assert ms.Predict(probe[:2]).tolist() == [int(ms.Labels()[0]), int(ms.Labels()[-1])]
    gm = ml.GaussianMixture(NComponents=2, Seed=0).Fit(X)
    pr = gm.PredictProba(probe[:2])
    assert pr.shape == (2, 2) and np.allclose(pr.sum(1), 1) and (pr.max(1) > 0.99).all()
    assert np.array_equal(gm.Predict(probe[:2]), pr.argmax(1))
    for clf in (ml.QDA().Fit(X, y), ml.AdaBoostClassifier(NEstimators=5, Seed=0).Fit(X, y)):
        pr = clf.PredictProba(probe[:2])
        assert pr.shape == (2, 2) and np.allclose(pr.sum(1), 1)
        assert np.array_equal(clf.Classes[pr.argmax(1)], clf.Predict(probe[:2])) and pr.argmax(1).tolist() == [0, 1]
    ts = ml.TSNE(NIter=50, Perplexity=5, Seed=0).Fit(X[::3])
    assert ts.Embedding.shape == (20, 2)


def test_exported_field_names_resolve_on_modules():
    lin, bn, mha = nn.Linear(3, 2), nn.BatchNorm1d(4), nn.MultiHeadAttention(8, 2)
    assert lin.Weight is lin.weight and lin.Bias is lin.bias and (lin.InFeatures, lin.OutFeatures) == (3, 2)
    assert bn.RunningMean is bn.running_mean and bn.Eps == 1e-5 and mha.NumHeads == 2 and mha.EmbedDim == 8
    with pytest.raises(AttributeError, match="no attribute 'Nope'"):
        lin.Nope
    assert not hasattr(lin, "WeightG")
    import copy, pickle
    assert torch.equal(copy.deepcopy(lin).Weight, lin.weight)
    assert torch.equal(pickle.loads(pickle.dumps(lin)).weight, lin.weight)


def test_round_to_dtype_known_patterns():
    """Rounding emulation against hand-checked IEEE values (round to nearest, ties to even)."""
    x = torch.tensor([0.1, 65504.0, 1e-8, 2049.0, 2051.0, 1.0 + 2 ** -11, 1.0 + 3 * 2 ** -11, -0.1], dtype=torch.float64)
    h = T.RoundTo(x, torch.float16)
    assert h.dtype == torch.float64
    assert h.tolist() == [0.0999755859375, 65504.0, 0.0, 2048.0, 2052.0, 1.0, 1.001953125, -0.0999755859375]
    f = T.RoundTo(torch.tensor([0.1, 16777217.0], dtype=torch.float64), torch.float32)
    assert f.tolist() == [0.10000000149011612, 16777216.0]
    b = T.RoundTo(torch.tensor([1.0 + 2 ** -8, 1.0 + 3 * 2 ** -8, 257.0, 259.0], dtype=torch.float64), torch.bfloat16)
    assert b.tolist() == [1.0, 1.015625, 256.0, 260.0]
    assert torch.equal(T.RoundTo(x, torch.float64), x)
    assert T.Promote(torch.float16, torch.float32) == torch.float32 and T.Promote(torch.float32, torch.float64) == torch.float64


def test_init_functions_take_the_reference_arguments():
    torch.manual_seed(0)
    w = torch.empty(64, 32, dtype=torch.float64)
    nn.XavierUniform(w, 32, 64)
    assert w.abs().max() <= math.sqrt(6 / 96) and w.std() > 0.1
    nn.KaimingNormal(w, 32)
    assert abs(float(w.std()) - math.sqrt(2 / 32)) < 0.02
    nn.KaimingUniform(w, 32)
    assert w.abs().max() <= math.sqrt(6 / 32)
    nn.XavierNormal(w)                                     # fans from the shape
    assert abs(float(w.std()) - math.sqrt(2 / 96)) < 0.01
    nn.Orthogonal(w[:32], 1.0)
    assert torch.allclose(w[:32] @ w[:32].t(), torch.eye(32, dtype=torch.float64), atol=1e-10)
    nn.Constant(w, 0.5)
    assert bool((w == 0.5).all())
    lin = nn.Linear(3, 2)
    assert [p.Name for p in nn.NamedParameters(lin)] == ["weight", "bias"]
    assert nn.FilterParams(lin, lambda name: name == "bias")[0] is lin.bias
    assert nn.FilterParams(lin, lambda name, p: p.dim() == 2)[0] is lin.weight
    assert ml.LinearDiscriminantAnalysis is ml.LDA and ml.QuadraticDiscriminantAnalysis is ml.QDA


def test_functional_options_become_keyword_arguments():
    c = nn.NewConv2d(3, 16, 3, nn.WithPadding(1), nn.WithStride(2), nn.WithNoBias(), nn.WithDilation(1, 1),
                     nn.WithGroups(1), nn.WithPaddingMode("reflect"))
    assert isinstance(c, nn.Conv2d) and c.padding == (1, 1) and c.stride == (2, 2) and c.bias is None
    t = nn.NewConvTranspose2d(4, 2, 3, nn.WithStride(2), nn.WithOutputPadding(1))
    assert t(torch.randn(1, 4, 5, 5)).shape == (1, 2, 12, 12)
    r = nn.NewLSTM(4, 8, nn.WithLayers(2), nn.WithBidirectional(), nn.WithProjSize(3))
    assert r.num_layers == 2 and r.bidirectional and r.proj_size == 3
    assert nn.NewRNN(4, 8, nn.WithReLU()).cells[0].relu if hasattr(nn.NewRNN(4, 8).cells[0], "relu") else True
    p = nn.NewMaxPool2d(2, nn.WithPoolStride(1), nn.WithPoolPadding(1), nn.WithPoolCeilMode(), nn.WithPoolDilation(1))
    assert p.stride == (1, 1) and p.padding == (1, 1) and p.ceil_mode
    assert not nn.NewAvgPool2d(3, nn.WithCountIncludePad(False)).count_include_pad
    bn = nn.NewBatchNorm2d(4, nn.WithEps(1e-3), nn.WithMomentum(0.2), nn.WithAffine(False))
    assert bn.eps == 1e-3 and bn.momentum == 0.2 and bn.weight is None
    e = nn.NewEmbedding(10, 4, nn.WithPaddingIdx(0), nn.WithMaxNorm(1.0))
    assert e.padding_idx == 0 and e.max_norm == 1.0
    assert nn.NewEmbeddingBag(10, 4, nn.WithBagMode("sum"), nn.WithBagPaddingIdx(1)).mode == "sum"
    enc = nn.NewTransformerEncoderLayer(8, 2, 16, nn.WithPreNorm(), nn.WithCausal(), nn.WithTransformerDropout(0.0))
    assert enc.pre_norm and enc.causal
    assert nn.NewMultiHeadAttention(8, 2, nn.WithKDim(6), nn.WithVDim(4)).kdim == 6
    l = nn.NewLocalResponseNorm(3, nn.WithLRNAlpha(1e-3), nn.WithLRNBeta(0.5), nn.WithLRNK(2.0))
    assert (l.alpha, l.beta, l.k) == (1e-3, 0.5, 2.0)
    assert nn.NewUpsample(2, "bilinear", nn.WithAlignCorners(True)).align_corners
    assert nn.NewSpectralNormLinear(nn.Linear(3, 3), nn.WithNPowerIterations(3), nn.WithSpectralEps(1e-9)).n_power_iterations == 3
    z, y = torch.randn(4, 5), torch.tensor([0, 1, 2, 1])
    got = nn.CrossEntropyLoss(z, y, nn.WithLabelSmoothing(0.1), nn.WithReduction(nn.ReduceSum), nn.WithIgnoreIndex(2))
    assert torch.equal(got, nn.CrossEntropyLoss(z, y, label_smoothing=0.1, reduction="sum", ignore_index=2))
    w = torch.nn.Parameter(torch.zeros(3))
    o = optim.NewSGD([w], 0.1, optim.WithMomentum(0.9), optim.WithNesterov(True), optim.WithSGDWeightDecay(0.01))
    assert (o.momentum, o.nesterov, o.Groups()[0].weight_decay) == (0.9, True, 0.01)
    a = optim.NewAdamW([w], 0.01, optim.WithAdamWBeta2(0.95), optim.WithAdamWWeightDecay(0.1), optim.WithAdamWEps(1e-6))
    assert (a.beta1, a.beta2) == (0.9, 0.95) and a.eps == 1e-6 and a.Groups()[0].weight_decay == 0.1
    rp = optim.NewRprop([w], 0.01, optim.WithRpropEtaMinus(0.4), optim.WithRpropStepBounds(1e-5, 10.0))
    assert (rp.eta_minus, rp.eta_plus, rp.step_min, rp.step_max) == (0.4, 1.2, 1e-5, 10.0)
    assert optim.NewASGD([w], 0.01, optim.WithASGDLambda(1e-3), optim.WithASGDT0(5.0)).lambd == 1e-3
    with pytest.raises(TypeError, match="no argument matches option WithStride"):
        nn.NewLinear(3, 2, nn.WithStride(2))
    with pytest.raises(AttributeError):
        nn.Withlowercase


def test_attention_call_options():
    m = nn.MultiHeadAttention(8, 2, dtype=torch.float64)
    q = torch.randn(2, 5, 8, dtype=torch.float64)
    pad = torch.zeros(2, 5, dtype=torch.bool)
    pad[1, 3:] = True
    mask = torch.triu(torch.ones(5, 5, dtype=torch.bool), 1)
    a = m.ForwardMasked(q, q, q, nn.WithCausal(), nn.WithKeyPaddingMask(pad))
    assert torch.equal(a, m.ForwardMasked(q, q, q, causal=True, key_padding_mask=pad))
    b = m.ForwardMasked(q, q, q, nn.WithAttnMask(mask))
    assert torch.allclose(b, m.ForwardMasked(q, q, q, causal=True), atol=1e-12)     # a causal mask given explicitly
    assert torch.allclose(b, m(q, q, q, True), atol=1e-6)


def test_group_constructors_accept_options():
    w, b = torch.nn.Parameter(torch.zeros(3)), torch.nn.Parameter(torch.zeros(2))
    o = optim.NewAdamWGroups([optim.Group([w], 1e-3, 0.1), optim.Group([b], 1e-3, 0.0)],
                             optim.WithAdamWBeta2(0.95), optim.WithAdamWEps(1e-6))
    assert (o.beta2, o.eps) == (0.95, 1e-6) and [g.weight_decay for g in o.Groups()] == [0.1, 0.0]
    with pytest.raises(TypeError):
        optim.NewSGDGroups([optim.Group([w], 0.1, 0.0)], 0.9)


def test_tensor_field_properties():
    x = T.SetRequiresGrad(T.New([1, 2, 3, 4, 5, 6], 2, 3))
    assert x.Shape == [2, 3] and x.Data.tolist() == [1, 2, 3, 4, 5, 6] and x.RequiresGrad and x.Grad is None
    x.Square().Sum().Backward()
    assert x.Grad.tolist() == [[2, 4, 6], [8, 10, 12]]
    x.Grad = None
    assert x.grad is None


def test_variadic_constructor_forms():
    assert nn.NewAdaptiveAvgPool2d(1, 1).output_size == (1, 1) and nn.AdaptiveAvgPool2d((2, 3)).output_size == (2, 3)
    assert nn.NewAdaptiveMaxPool3d(1, 2, 3).output_size == (1, 2, 3) and nn.AdaptiveMaxPool1d(3).output_size == (3,)
    with pytest.raises(ValueError):
        nn.NewAdaptiveAvgPool2d(1, 2, 3)
    assert nn.NewParameterList(torch.zeros(2), torch.ones(3)).Len() == 2
    assert nn.NewModuleList(nn.ReLU(), nn.Tanh()).Len() == 2 and nn.NewModuleList([nn.ReLU()]).Len() == 1
    assert nn.NewUnflatten(1, 2, 3)(torch.zeros(4, 6)).shape == (4, 2, 3)
    assert nn.NewSequential(nn.NewLinear(2, 3, True), nn.ReLU())(torch.zeros(1, 2)).shape == (1, 3)
    x = torch.randn(1, 2, 10, 10)
    fp = nn.NewFractionalMaxPool2d(2, nn.WithOutputRatio(0.5, 0.7), nn.WithFractionalSamples(0.3, 0.6))
    assert fp(x).shape == (1, 2, 5, 7)
    assert nn.NewFractionalMaxPool2d(2, nn.WithOutputSize(4, 4))(x).shape == (1, 2, 4, 4)
    with pytest.raises(ValueError):
        nn.NewFractionalMaxPool2d(2)
    assert nn.NewFold((4, 4), 2, nn.WithStride(2))(torch.randn(1, 8, 4)).shape == (1, 2, 4, 4)
    assert nn.NewUnfold(2, nn.WithStride(2))(torch.randn(1, 2, 4, 4)).shape == (1, 8, 4)
    assert nn.NewLPPool2d(2.0, 2)(x.abs()).shape == (1, 2, 5, 5)


def test_estimator_result_fields_under_the_reference_names():
    rng = np.random.default_rng(0)
    x = rng.random((100, 1)) * 10
    y = 2.5 * x[:, 0] + 1.7 + rng.normal(0, 0.05, 100)
    lr = ml.LinearRegression().Fit(x, y)
    assert abs(lr.Weights[0] - 2.5) < 0.02 and abs(lr.Bias - 1.7) < 0.1
    X = np.concatenate([rng.normal(0, 0.3, (30, 2)), rng.normal(3, 0.3, (30, 2))])
    lab = np.array([0] * 30 + [1] * 30)
    km = ml.KMeans(K=2, Seed=1).Fit(X)
    assert np.asarray(km.Centroids).shape == (2, 2) and km.Centroids is km.Centers
    lg = ml.LogisticRegression(MaxIter=200).Fit(X, lab)
    assert np.asarray(lg.Weights).shape == (2, 2) and np.asarray(lg.Bias).shape == (2,)
    z = X @ np.asarray(lg.Weights).T + np.asarray(lg.Bias)
    assert np.array_equal(z.argmax(1), lg.Predict(X))
    knn = ml.KNNClassifier(K=3).Fit(X, lab)
    assert np.asarray(knn.Xtrain).shape == (60, 2) and np.asarray(knn.Ytrain).shape == (60,)
    gm = ml.GaussianMixture(NComponents=2, Seed=0).Fit(X)
    assert np.asarray(gm.Covariances).shape == (2, 2) and np.isfinite(gm.LogLikelihood)
    br = ml.BayesianRidge().Fit(x, y)
    assert br.AlphaPrec > 0 and br.LambdaPrec > 0 and abs(br.Weights[0] - 2.5) < 0.05
    assert np.asarray(ml.LDA(NComponents=1).Fit(X, lab).Components).shape == (1, 2)
    assert np.asarray(ml.FastICA(NComponents=2, Seed=0).Fit(X).Components).shape == (2, 2)
    assert ml.OneHotEncoder().Fit(np.array([2, 0, 1, 2])).Classes.tolist() == [0, 1, 2]
    with pytest.raises(AttributeError):
        ml.KMeans(K=2).Centroids                      # nothing fitted yet


def test_module_field_aliases_and_embedding_bag_max_norm():
    assert nn.Bilinear(3, 4, 5).In1Features == 3 and nn.Unfold(2, stride=2).Kernel == (2, 2)
    assert nn.AdaptiveAvgPool2d((2, 3)).OutH == 2 and nn.AdaptiveAvgPool2d((2, 3)).OutW == 3
    p = nn.ReflectionPad2d(1, 2, 3, 4)
    assert (p.Top, p.Bottom, p.Left, p.Right) == (1, 2, 3, 4)
    p3 = nn.CircularPad3d(1, 2, 3, 4, 5, 6)
    assert (p3.Left, p3.Right, p3.Top, p3.Bottom, p3.Front, p3.Back) == (1, 2, 3, 4, 5, 6)
    wn = nn.WeightNormLinear(nn.Linear(3, 2))
    assert wn.G is wn.weight_g and wn.V is wn.weight_v and (wn.InFeatures, wn.OutFeatures) == (3, 2)
    assert nn.Softmax(-1).Axis == -1 and nn.Upsample(3).ScaleFactor == 3 and nn.PixelShuffle(2).UpscaleFactor == 2
    als = nn.AdaptiveLogSoftmaxWithLoss(8, 12, [4, 8], div_value=2.0)
    assert (als.ShortlistSize, als.HeadSize, als.DivValue, als.HeadBias) == (4, 6, 2.0, False)
    torch.manual_seed(0)
    eb = nn.NewEmbeddingBag(10, 4, nn.WithBagMode("sum"), nn.WithBagMaxNorm(0.5), nn.WithDType(torch.float64))
    eb(torch.tensor([[1, 2], [3, 3]]))
    norms = eb.weight.detach().norm(dim=1)
    assert torch.allclose(norms[1:4], torch.full((3,), 0.5, dtype=torch.float64), atol=1e-6) and norms[5] > 0.5
    assert eb.MaxNorm == 0.5


def test_synthetic_generators_take_the_reference_arguments():
    X, Y = data.MakeClassification(100, 20, 3, 42)               # samples, features, classes, seed
    assert X.shape == (100, 20) and set(Y.tolist()) <= {0, 1, 2}
    X2, _ = data.MakeClassification(100, 20, 3, 42)
    assert torch.equal(X, X2) and not torch.equal(X, data.MakeClassification(100, 20, 3, 43)[0])
    Xb, yb = data.MakeBlobs(60, 2, 3, 7)
    assert Xb.shape == (60, 2) and torch.equal(Xb, data.MakeBlobs(60, 2, 3, seed=7)[0])
    Xr, yr = data.MakeRegression(50, 4, 0.1, 5)
    assert Xr.shape == (50, 4) and yr.shape == (50,) and data.MakeRegression(50, 4, 0.1, 5).Weights.shape == (4,)
    Xm, ym = data.MakeMoons(40, 0.05, 1)
    assert Xm.shape == (40, 2) and ym.sum() == 20
    loader = data.NewDataLoader(data.NewTensorDataset(X, Y), 32, True)
    shapes = [tuple(b.X.shape) for b in loader.Iter()]
    assert shapes == [(32, 20)] * 3 + [(4, 20)] and loader.Len() == 4


def test_option_overrides_the_positional_value():
    c = nn.NewConv2d(3, 8, 3, nn.WithKernel(3, 5), nn.WithStride(1, 2), nn.WithPad(1, 2))
    assert c.kernel_size == (3, 5) and c.stride == (1, 2) and c.padding == (1, 2)
    assert c(torch.randn(1, 3, 8, 8)).shape == (1, 8, 8, 4)

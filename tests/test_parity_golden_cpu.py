"""Golden parity file: one instance of every module family, seeded, recorded as parameter
count / shapes and output shape / sum / first three values at 12 significant digits, and
compared byte for byte with ``tests/testdata/parity.golden`` (the reference keeps the same
kind of file, nn/parity_test.go:56-400).  Regenerate with ``GONN_UPDATE_GOLDEN=1``."""
import os

import torch

from gonn_b200 import nn

GOLDEN = os.path.join(os.path.dirname(__file__), "testdata", "parity.golden")
D = torch.float64


def _inp(*shape):
    return torch.randn(*shape, dtype=D)


def _idx(n, *shape):
    return torch.randint(0, n, shape)


CASES = [
    ("Linear", lambda: nn.Linear(5, 4, dtype=D), lambda: (_inp(3, 5),)),
    ("Bilinear", lambda: nn.Bilinear(3, 4, 5, dtype=D), lambda: (_inp(2, 3), _inp(2, 4))),
    ("Conv1d", lambda: nn.Conv1d(2, 3, 3, padding=1, dtype=D), lambda: (_inp(2, 2, 7),)),
    ("Conv2d", lambda: nn.Conv2d(2, 3, 3, stride=2, padding=1, dtype=D), lambda: (_inp(2, 2, 6, 5),)),
    ("Conv3d", lambda: nn.Conv3d(1, 2, 2, dtype=D), lambda: (_inp(1, 1, 3, 4, 3),)),
    ("ConvTranspose1d", lambda: nn.ConvTranspose1d(2, 3, 3, stride=2, dtype=D), lambda: (_inp(1, 2, 4),)),
    ("ConvTranspose2d", lambda: nn.ConvTranspose2d(2, 3, 3, stride=2, dtype=D), lambda: (_inp(1, 2, 3, 3),)),
    ("ConvTranspose3d", lambda: nn.ConvTranspose3d(1, 2, 2, dtype=D), lambda: (_inp(1, 1, 2, 3, 2),)),
    ("Unfold", lambda: nn.Unfold(2, stride=1), lambda: (_inp(1, 2, 3, 4),)),
    ("MaxPool2d", lambda: nn.MaxPool2d(2), lambda: (_inp(1, 2, 4, 6),)),
    ("AvgPool2d", lambda: nn.AvgPool2d(3, 2, 1, ceil_mode=True), lambda: (_inp(1, 2, 6, 6),)),
    ("LPPool2d", lambda: nn.LPPool2d(2.0, 2), lambda: (_inp(1, 2, 4, 4),)),
    ("AdaptiveAvgPool2d", lambda: nn.AdaptiveAvgPool2d((2, 3)), lambda: (_inp(1, 2, 5, 7),)),
    ("AdaptiveMaxPool1d", lambda: nn.AdaptiveMaxPool1d(3), lambda: (_inp(1, 2, 8),)),
    ("FractionalMaxPool2d", lambda: nn.FractionalMaxPool2d(2, 3, samples=[0.25, 0.75]), lambda: (_inp(1, 1, 7, 7),)),
    ("LayerNorm", lambda: nn.LayerNorm(6, dtype=D), lambda: (_inp(4, 6),)),
    ("RMSNorm", lambda: nn.RMSNorm(6, dtype=D), lambda: (_inp(4, 6),)),
    ("BatchNorm1d", lambda: nn.BatchNorm1d(4, dtype=D), lambda: (_inp(6, 4),)),
    ("BatchNorm2d", lambda: nn.BatchNorm2d(3, dtype=D), lambda: (_inp(4, 3, 3, 2),)),
    ("GroupNorm", lambda: nn.GroupNorm(2, 4, dtype=D), lambda: (_inp(2, 4, 3),)),
    ("InstanceNorm2d", lambda: nn.InstanceNorm2d(3), lambda: (_inp(2, 3, 4, 4),)),
    ("LocalResponseNorm", lambda: nn.LocalResponseNorm(3), lambda: (_inp(2, 4, 3),)),
    ("Embedding", lambda: nn.Embedding(10, 4, dtype=D), lambda: (_idx(10, 2, 5),)),
    ("EmbeddingBag", lambda: nn.EmbeddingBag(10, 4, "mean", dtype=D), lambda: (_idx(10, 3, 4),)),
    ("RNN", lambda: nn.RNN(3, 4, dtype=D), lambda: (_inp(2, 5, 3),)),
    ("LSTM", lambda: nn.LSTM(3, 4, num_layers=2, bidirectional=True, dtype=D), lambda: (_inp(2, 5, 3),)),
    ("GRU", lambda: nn.GRU(3, 4, dtype=D), lambda: (_inp(2, 5, 3),)),
    ("MultiHeadAttention", lambda: nn.MultiHeadAttention(8, 2, dtype=D), lambda: (_inp(2, 5, 8),)),
    ("TransformerEncoderLayer", lambda: nn.TransformerEncoderLayer(8, 2, 16, dtype=D).eval(), lambda: (_inp(2, 5, 8),)),
    ("TransformerDecoderLayer", lambda: nn.TransformerDecoderLayer(8, 2, 16, dtype=D).eval(),
     lambda: (_inp(2, 4, 8), _inp(2, 5, 8))),
    ("Transformer", lambda: nn.Transformer(8, 2, 1, 1, 16, dtype=D).eval(), lambda: (_inp(2, 5, 8), _inp(2, 4, 8))),
    ("PReLU", lambda: nn.PReLU(dtype=D), lambda: (_inp(3, 4),)),
    ("GLU", lambda: nn.GLU(), lambda: (_inp(3, 6),)),
    ("GELU", lambda: nn.GELU(), lambda: (_inp(3, 4),)),
    ("Mish", lambda: nn.Mish(), lambda: (_inp(3, 4),)),
    ("Softmax", lambda: nn.Softmax(-1), lambda: (_inp(3, 5),)),
    ("ReflectionPad2d", lambda: nn.ReflectionPad2d(1, 2, 2, 1), lambda: (_inp(1, 2, 4, 4),)),
    ("CircularPad3d", lambda: nn.CircularPad3d(1, 0, 1, 1, 0, 1), lambda: (_inp(1, 1, 2, 3, 3),)),
    ("Upsample", lambda: nn.Upsample(2, "bicubic"), lambda: (_inp(1, 2, 3, 3),)),
    ("PixelShuffle", lambda: nn.PixelShuffle(2), lambda: (_inp(1, 8, 2, 3),)),
    ("WeightNormLinear", lambda: nn.WeightNormLinear(nn.Linear(5, 4, dtype=D)), lambda: (_inp(3, 5),)),
    ("SpectralNormLinear", lambda: nn.SpectralNormLinear(nn.Linear(5, 4, dtype=D)).eval(), lambda: (_inp(3, 5),)),
    ("AdaptiveLogSoftmaxWithLoss.LogProb", lambda: nn.AdaptiveLogSoftmaxWithLoss(8, 12, [4, 8], dtype=D), lambda: (_inp(3, 8),)),
]


def _fmt(v: float) -> str:
    return "%.12g" % (0.0 if v == 0 else v)


def _record(name, make, inputs) -> str:
    torch.manual_seed(20240607)
    m = make()
    xs = inputs()
    with torch.no_grad():
        fn = m.LogProb if name.endswith(".LogProb") else m
        y = fn(*xs)
    if isinstance(y, tuple):
        y = y[0]
    ps = list(m.parameters())
    shapes = ";".join("x".join(str(d) for d in p.shape) for p in ps)
    flat = y.reshape(-1).double()
    first = ",".join(_fmt(float(v)) for v in flat[:3])
    return (f"{name} params={sum(p.numel() for p in ps)} shapes=[{shapes}] out={'x'.join(str(d) for d in y.shape)} "
            f"sum={_fmt(float(flat.sum()))} first=[{first}]")


def test_parity_golden():
    lines = [_record(*c) for c in CASES]
    text = "\n".join(lines) + "\n"
    if os.environ.get("GONN_UPDATE_GOLDEN") == "1" or not os.path.exists(GOLDEN):
        with open(GOLDEN, "w", newline="\n") as f:
            f.write(text)
    with open(GOLDEN, newline="") as f:
        want = f.read()
    got_lines, want_lines = text.splitlines(), want.splitlines()
    assert len(got_lines) == len(want_lines), "module list changed: regenerate with GONN_UPDATE_GOLDEN=1"
    for g, w in zip(got_lines, want_lines):
        assert g == w
    # recording twice gives the same bytes (seeding covers construction and inputs)
    assert _record(*CASES[0]) == lines[0]

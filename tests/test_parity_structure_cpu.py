"""Structure of every module family against the reference's golden file.

The reference records, for one seeded instance of each module family, the number of
parameters, every parameter's shape in registration order, and the output shape for a fixed
input (nn/testdata/parity.golden, written by nn/parity_test.go:56-400).  The random values
come from Go's generator and cannot be reproduced here, but the structure can: the table
below holds the structural fields of that file (name, parameter shapes, output shape), and
each entry is built with this package's constructor and fed an input of the reference's shape.
"""
import pytest
import torch

from gonn_b200 import nn

D = torch.float64


def r(*shape):
    return torch.randn(*shape, dtype=D)


# name in the reference's golden file, constructor, inputs, parameter shapes, output shape
TABLE = [
    ("Linear(4,3,bias)", lambda: nn.Linear(4, 3, True, dtype=D), lambda: (r(2, 4),), [[3, 4], [3]], [2, 3]),
    ("Linear(4,3,nobias)", lambda: nn.Linear(4, 3, False, dtype=D), lambda: (r(2, 4),), [[3, 4]], [2, 3]),
    ("Conv1d(2,3,k3,s2,p1)", lambda: nn.Conv1d(2, 3, 3, stride=2, padding=1, dtype=D), lambda: (r(2, 2, 7),),
     [[3, 2, 3], [3]], [2, 3, 4]),
    ("Conv2d(2,3,k3,s2,p1)", lambda: nn.Conv2d(2, 3, 3, stride=2, padding=1, dtype=D), lambda: (r(2, 2, 6, 7),),
     [[3, 2, 3, 3], [3]], [2, 3, 3, 4]),
    ("Conv2dHW(2,3,k32,s21,p10)", lambda: nn.Conv2d(2, 3, (3, 2), stride=(2, 1), padding=(1, 0), dtype=D),
     lambda: (r(2, 2, 6, 7),), [[3, 2, 3, 2], [3]], [2, 3, 3, 6]),
    ("Conv3d(2,2,k2,s1,p0)", lambda: nn.Conv3d(2, 2, 2, dtype=D), lambda: (r(2, 2, 3, 4, 4),),
     [[2, 2, 2, 2, 2], [2]], [2, 2, 2, 3, 3]),
    ("ConvTranspose1d(2,3,k3,s2,p1)", lambda: nn.ConvTranspose1d(2, 3, 3, stride=2, padding=1, dtype=D),
     lambda: (r(2, 2, 5),), [[2, 3, 3], [3]], [2, 3, 9]),
    ("ConvTranspose2d(2,3,k3,s2,p1)", lambda: nn.ConvTranspose2d(2, 3, 3, stride=2, padding=1, dtype=D),
     lambda: (r(2, 2, 4, 4),), [[2, 3, 3, 3], [3]], [2, 3, 7, 7]),
    ("ConvTranspose3d(2,2,k2,s2,p0)", lambda: nn.ConvTranspose3d(2, 2, 2, stride=2, dtype=D),
     lambda: (r(1, 2, 3, 3, 3),), [[2, 2, 2, 2, 2], [2]], [1, 2, 6, 6, 6]),
    ("MaxPool1d(2,2)", lambda: nn.MaxPool1d(2), lambda: (r(2, 2, 6),), [], [2, 2, 3]),
    ("AvgPool1d(2,2)", lambda: nn.AvgPool1d(2), lambda: (r(2, 2, 6),), [], [2, 2, 3]),
    ("MaxPool2d(2,2)", lambda: nn.MaxPool2d(2), lambda: (r(2, 2, 4, 4),), [], [2, 2, 2, 2]),
    ("AvgPool2d(2,2)", lambda: nn.AvgPool2d(2), lambda: (r(2, 2, 4, 4),), [], [2, 2, 2, 2]),
    ("MaxPool3d(2,2)", lambda: nn.MaxPool3d(2), lambda: (r(1, 2, 4, 4, 4),), [], [1, 2, 2, 2, 2]),
    ("AvgPool3d(2,2)", lambda: nn.AvgPool3d(2), lambda: (r(1, 2, 4, 4, 4),), [], [1, 2, 2, 2, 2]),
    ("AdaptiveAvgPool1d(3)", lambda: nn.AdaptiveAvgPool1d(3), lambda: (r(2, 2, 7),), [], [2, 2, 3]),
    ("AdaptiveMaxPool2d(2,2)", lambda: nn.AdaptiveMaxPool2d((2, 2)), lambda: (r(2, 2, 5, 5),), [], [2, 2, 2, 2]),
    ("AdaptiveAvgPool2d(2,2)", lambda: nn.AdaptiveAvgPool2d((2, 2)), lambda: (r(2, 2, 5, 5),), [], [2, 2, 2, 2]),
    ("AdaptiveAvgPool3d(2,2,2)", lambda: nn.AdaptiveAvgPool3d((2, 2, 2)), lambda: (r(1, 2, 4, 4, 4),), [],
     [1, 2, 2, 2, 2]),
    ("LayerNorm(6)", lambda: nn.LayerNorm(6, dtype=D), lambda: (r(3, 6),), [[6], [6]], [3, 6]),
    ("RMSNorm(6)", lambda: nn.RMSNorm(6, dtype=D), lambda: (r(3, 6),), [[6]], [3, 6]),
    ("BatchNorm1d(4)-train", lambda: nn.BatchNorm1d(4, dtype=D), lambda: (r(5, 4),), [[4], [4]], [5, 4]),
    ("BatchNorm1d(4)-eval", lambda: nn.BatchNorm1d(4, dtype=D).eval(), lambda: (r(5, 4),), [[4], [4]], [5, 4]),
    ("BatchNorm2d(3)-train", lambda: nn.BatchNorm2d(3, dtype=D), lambda: (r(2, 3, 4, 4),), [[3], [3]], [2, 3, 4, 4]),
    ("GroupNorm(2,4)", lambda: nn.GroupNorm(2, 4, dtype=D), lambda: (r(2, 4, 5),), [[4], [4]], [2, 4, 5]),
    ("InstanceNorm1d(2,affine)", lambda: nn.InstanceNorm1d(2, affine=True, dtype=D), lambda: (r(2, 2, 6),),
     [[2], [2]], [2, 2, 6]),
    ("InstanceNorm2d(2,noaffine)", lambda: nn.InstanceNorm2d(2), lambda: (r(2, 2, 4, 4),), [], [2, 2, 4, 4]),
    ("Embedding(5,3)", lambda: nn.Embedding(5, 3, dtype=D), lambda: (torch.tensor([0, 2, 4, 1]),), [[5, 3]], [4, 3]),
    ("PReLU(3)", lambda: nn.PReLU(3, dtype=D), lambda: (r(2, 3, 4),), [[3]], [2, 3, 4]),
    ("GLU(dim=-1)", lambda: nn.GLU(-1), lambda: (r(3, 8),), [], [3, 4]),
    ("Bilinear(3,4,2,bias)", lambda: nn.Bilinear(3, 4, 2, dtype=D), lambda: (r(2, 3), r(2, 4)), [[2, 3, 4], [2]], [2, 2]),
    ("Flatten(1,-1)", lambda: nn.Flatten(1, -1), lambda: (r(2, 3, 4),), [], [2, 12]),
    ("Unflatten(1,[2,3])", lambda: nn.Unflatten(1, (2, 3)), lambda: (r(2, 6),), [], [2, 2, 3]),
    ("CosineSimilarity(1)", lambda: nn.CosineSimilarity(1, 1e-8), lambda: (r(3, 4), r(3, 4)), [], [3]),
    ("PairwiseDistance(2)", lambda: nn.PairwiseDistance(2, 1e-8), lambda: (r(3, 4), r(3, 4)), [], [3]),
    ("ZeroPad2d(1,1,1,1)", lambda: nn.ZeroPad2d(1, 1, 1, 1), lambda: (r(1, 2, 3, 3),), [], [1, 2, 5, 5]),
    ("ConstantPad2d(1,0,2,1,v=2.5)", lambda: nn.ConstantPad2d(1, 0, 2, 1, 2.5), lambda: (r(1, 2, 3, 3),), [],
     [1, 2, 4, 6]),
    ("ReflectionPad2d(1,1,1,1)", lambda: nn.ReflectionPad2d(1, 1, 1, 1), lambda: (r(1, 2, 3, 3),), [], [1, 2, 5, 5]),
    ("ReplicationPad2d(2,1,1,2)", lambda: nn.ReplicationPad2d(2, 1, 1, 2), lambda: (r(1, 2, 3, 3),), [],
     [1, 2, 6, 6]),
    ("Upsample(2,nearest)", lambda: nn.Upsample(scale_factor=2, mode="nearest"), lambda: (r(1, 2, 3, 3),), [],
     [1, 2, 6, 6]),
    ("Upsample(2,bilinear)", lambda: nn.Upsample(scale_factor=2, mode="bilinear"), lambda: (r(1, 2, 3, 3),), [],
     [1, 2, 6, 6]),
    ("PixelShuffle(2)", lambda: nn.PixelShuffle(2), lambda: (r(1, 8, 3, 3),), [], [1, 2, 6, 6]),
    ("PixelUnshuffle(2)", lambda: nn.PixelUnshuffle(2), lambda: (r(1, 2, 6, 6),), [], [1, 8, 3, 3]),
    ("RNN(3,4)", lambda: nn.RNN(3, 4, dtype=D), lambda: (r(2, 3, 3),), [[4, 3], [4], [4, 4]], [2, 3, 4]),
    ("LSTM(3,4)", lambda: nn.LSTM(3, 4, dtype=D), lambda: (r(2, 3, 3),), [[16, 3], [16], [16, 4]], [2, 3, 4]),
    ("GRU(3,4)", lambda: nn.GRU(3, 4, dtype=D), lambda: (r(2, 3, 3),), [[12, 3], [12], [12, 4], [12]], [2, 3, 4]),
    ("MultiLayerRNN(3,4,2,bidir)", lambda: nn.RNN(3, 4, num_layers=2, bidirectional=True, dtype=D),
     lambda: (r(2, 3, 3),), [[4, 3], [4], [4, 4], [4, 8], [4], [4, 4]] * 2,
     [2, 3, 8]),
    ("MultiLayerLSTM(3,4,2)", lambda: nn.LSTM(3, 4, num_layers=2, dtype=D), lambda: (r(2, 3, 3),),
     [[16, 3], [16], [16, 4], [16, 4], [16], [16, 4]], [2, 3, 4]),
    ("MultiLayerGRU(3,4,2,bidir)", lambda: nn.GRU(3, 4, num_layers=2, bidirectional=True, dtype=D),
     lambda: (r(2, 3, 3),),
     [[12, 3], [12], [12, 4], [12], [12, 8], [12], [12, 4], [12]] * 2, [2, 3, 8]),
    ("MultiHeadAttention(8,2)-causal", lambda: nn.MultiHeadAttention(8, 2, dtype=D), "mha",
     [[8, 8], [8]] * 4, [2, 3, 8]),
    ("TransformerEncoderLayer(8,2,16)", lambda: nn.TransformerEncoderLayer(8, 2, 16, dtype=D).eval(),
     lambda: (r(2, 3, 8),), [[8, 8], [8]] * 4 + [[8], [8], [16, 8], [16], [8, 16], [8], [8], [8]], [2, 3, 8]),
    ("TransformerEncoder(2,8,2,16)", lambda: nn.TransformerEncoder(2, 8, 2, 16, dtype=D).eval(),
     lambda: (r(2, 3, 8),), ([[8, 8], [8]] * 4 + [[8], [8], [16, 8], [16], [8, 16], [8], [8], [8]]) * 2, [2, 3, 8]),
    ("TransformerDecoderLayer(8,2,16)", lambda: nn.TransformerDecoderLayer(8, 2, 16, dtype=D).eval(),
     lambda: (r(2, 3, 8), r(2, 4, 8)),
     [[8, 8], [8]] * 4 + [[8], [8]] + [[8, 8], [8]] * 4 + [[8], [8], [16, 8], [16], [8, 16], [8], [8], [8]], [2, 3, 8]),
    ("Seq2Seq(5,6,4,8)", lambda: nn.Seq2Seq(5, 6, 4, 8, dtype=D), "seq2seq",
     [[5, 4], [6, 4], [32, 4], [32], [32, 8], [32, 4], [32], [32, 8], [6, 8], [6]], [2, 2, 6]),
    ("Sequential(Lin-ReLU-Lin)", lambda: nn.Sequential(nn.Linear(4, 8, dtype=D), nn.ReLU(), nn.Linear(8, 2, dtype=D)),
     lambda: (r(3, 4),), [[8, 4], [8], [2, 8], [2]], [3, 2]),
    ("Softmax(axis1)", lambda: nn.Softmax(1), lambda: (r(3, 5),), [], [3, 5]),
    ("GELU-module", lambda: nn.GELU(), lambda: (r(3, 5),), [], [3, 5]),
    ("SiLU-module", lambda: nn.SiLU(), lambda: (r(3, 5),), [], [3, 5]),
]


def test_table_covers_every_line_of_the_reference_golden():
    # the reference's file has 58 entries; the table restates each one's structural fields
    assert len(TABLE) == 58
    assert len({t[0] for t in TABLE}) == 58


@pytest.mark.parametrize("name,make,inputs,param_shapes,out_shape", TABLE, ids=[t[0] for t in TABLE])
def test_structure_matches_reference(name, make, inputs, param_shapes, out_shape):
    torch.manual_seed(0)
    m = make()
    if inputs == "mha":
        x = r(2, 3, 8)
        out = m(x, x, x, True)
    elif inputs == "seq2seq":
        out = m(torch.tensor([[0, 1, 2], [3, 4, 0]]), torch.tensor([[0, 1], [2, 3]]))
    else:
        out = m(*inputs())
    if isinstance(out, tuple):
        out = out[0]
    got = [list(p.shape) for p in m.parameters()]
    assert len(got) == len(param_shapes), (name, got)
    assert sorted(got) == sorted(param_shapes), (name, got)
    assert got == param_shapes, f"{name}: same shapes, different registration order {got}"
    assert list(out.shape) == out_shape, (name, list(out.shape))

"""The MLP example written in the reference's own spelling (examples/mlp/main.go): constructor
functions, methods on tensors and modules, exported field names.  It runs unchanged apart from
the syntax of the language, which is the point: code that was written against GoNN's API reads
the same here.  The one addition is ``nn.WithDType``: the reference computes in float64 throughout,
here layers default to float32 and are told to match the data.  Idiomatic use of this framework
is in ``mlp.py``."""
import math
import os
import random
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from gonn_b200 import nn, optim, tensor  # noqa: E402


def make_blobs(n, classes):
    """(X, y): X (n, 2), y (n,) class ids stored as float64, three clusters on a circle."""
    x_data, y_data = [], []
    for i in range(n):
        c = i % classes
        ang = c * 2 * math.pi / classes
        x_data += [3 * math.cos(ang) + random.gauss(0, 0.5), 3 * math.sin(ang) + random.gauss(0, 0.5)]
        y_data.append(float(c))
    return tensor.New(x_data, n, 2), tensor.New(y_data, n)


def accuracy(logits, targets):
    preds = logits.ArgMax(1)
    correct = sum(1 for p, t in zip(preds.Data.tolist(), targets.Data.tolist()) if int(p) == int(t))
    return correct / targets.Numel()


def main(epochs: int = 200, verbose: bool = True):
    random.seed(7)
    torch.manual_seed(7)
    X, Y = make_blobs(300, 3)
    model = nn.NewSequential(
        nn.NewLinear(2, 32, True, nn.WithDType(X.DType())),
        nn.ReLU(),
        nn.NewLinear(32, 16, True, nn.WithDType(X.DType())),
        nn.ReLU(),
        nn.NewLinear(16, 3, True, nn.WithDType(X.DType())),
    )
    opt = optim.NewAdam(model.Parameters(), 0.01)
    for epoch in range(epochs):
        opt.ZeroGrad()
        logits = model.Forward(X)
        loss = nn.CrossEntropyLoss(logits, Y)
        loss.Backward()
        opt.Step()
        if verbose and epoch % 20 == 0:
            print(f"epoch {epoch:3d}  loss={float(loss.Data[0]):.4f}  acc={accuracy(logits, Y) * 100:.2f}%")
    final = accuracy(model.Forward(X), Y)
    if verbose:
        print(f"\nfinal accuracy = {final * 100:.2f}%")
    return final


if __name__ == "__main__":
    main()

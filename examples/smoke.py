"""Smoke demo (the reference's main.go): a tensor round trip through the op registry, one
layer, one backward pass and one optimizer step, on the GPU when there is one."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from gonn_b200 import nn, optim, tensor  # noqa: E402


def main():
    device = "cuda" if torch.cuda.is_available() else "cpu"
    x = torch.randn(4, 8, device=device)
    print("registered unary ops:", ", ".join(sorted(tensor.UnaryOpNames())[:8]), "...")
    print("tanh(x)[0,:3] =", tensor.Unary(x, "tanh")[0, :3].tolist())
    layer = nn.Linear(8, 3, device=device)
    opt = optim.SGD(layer.parameters(), lr=0.1, momentum=0.9)
    loss = nn.MSELoss(layer(x), torch.zeros(4, 3, device=device))
    loss.backward()
    opt.step()
    print(f"device {device}: loss {loss.item():.4f}, |grad W| {layer.weight.grad.norm().item():.4f}")


if __name__ == "__main__":
    main()

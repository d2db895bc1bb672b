"""Linear regression with SGD (the reference's examples/regression/main.go): fits
y = X w + b on synthetic data and prints the loss every 20 steps."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from gonn_b200 import nn, optim  # noqa: E402
from gonn_b200.data import MakeRegression  # noqa: E402


def main(steps: int = 200, device: str = "cpu"):
    X, y = MakeRegression(256, 8, noise=0.05, seed=1)
    X, y = X.to(device), y.to(device).reshape(-1, 1)
    model = nn.Linear(8, 1, dtype=X.dtype, device=device)
    opt = optim.SGD(model.parameters(), lr=0.05)
    loss = None
    for step in range(steps):
        opt.zero_grad()
        loss = nn.MSELoss(model(X), y)
        loss.backward()
        opt.step()
        if step % 20 == 0:
            print(f"step {step:4d}  mse {loss.item():.5f}")
    return float(loss.item())


if __name__ == "__main__":
    main(device="cuda" if torch.cuda.is_available() else "cpu")

"""Three-class classification of Gaussian blobs with an MLP and Adam (the reference's
examples/mlp/main.go)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from gonn_b200 import nn, optim  # noqa: E402
from gonn_b200.data import DataLoader, MakeBlobs, TensorDataset  # noqa: E402


def main(epochs: int = 20, device: str = "cpu"):
    X, y = MakeBlobs(300, 2, centers=3, std=0.6, seed=0)
    X = X.to(torch.float32)
    model = nn.Sequential(nn.Linear(2, 32, device=device), nn.ReLU(), nn.Linear(32, 3, device=device))
    opt = optim.Adam(model.parameters(), lr=0.01)
    loader = DataLoader(TensorDataset(X, y), batch_size=32, shuffle=True, seed=0)
    acc = 0.0
    for epoch in range(epochs):
        for xb, yb in loader:
            xb, yb = xb.to(device), yb.to(device)
            opt.zero_grad()
            loss = nn.CrossEntropyLoss(model(xb), yb)
            loss.backward()
            opt.step()
        with torch.no_grad():
            acc = (model(X.to(device)).argmax(1).cpu() == y).float().mean().item()
        if epoch % 5 == 0:
            print(f"epoch {epoch:3d}  loss {loss.item():.4f}  accuracy {acc:.3f}")
    return acc


if __name__ == "__main__":
    main(device="cuda" if torch.cuda.is_available() else "cpu")

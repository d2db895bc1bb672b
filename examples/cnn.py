"""Small CNN on synthetic 1x8x8 images (the reference's examples/cnn/main.go):
Conv - ReLU - MaxPool - Conv - ReLU - global average pool - Linear."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from gonn_b200 import nn, optim  # noqa: E402


class Net(nn.Module):
    def __init__(self, device):
        super().__init__()
        self.c1 = nn.Conv2d(1, 8, 3, padding=1, device=device)
        self.c2 = nn.Conv2d(8, 16, 3, padding=1, device=device)
        self.pool = nn.MaxPool2d(2)
        self.gap = nn.AdaptiveAvgPool2d(1)
        self.fc = nn.Linear(16, 2, device=device)
        self.act = nn.ReLU()

    def forward(self, x):
        x = self.pool(self.act(self.c1(x)))
        x = self.gap(self.act(self.c2(x)))
        return self.fc(x.flatten(1))


def main(steps: int = 60, device: str = "cpu"):
    g = torch.Generator().manual_seed(0)
    # class 1 images have a bright top-left quadrant
    x = torch.randn(64, 1, 8, 8, generator=g) * 0.3
    y = torch.randint(0, 2, (64,), generator=g)
    x[y == 1, :, :4, :4] += 1.0
    x, y = x.to(device), y.to(device)
    model = Net(device)
    opt = optim.Adam(model.parameters(), lr=0.02)
    acc = 0.0
    for step in range(steps):
        opt.zero_grad()
        logits = model(x)
        loss = nn.CrossEntropyLoss(logits, y)
        loss.backward()
        opt.step()
        acc = (logits.argmax(1) == y).float().mean().item()
        if step % 10 == 0:
            print(f"step {step:3d}  loss {loss.item():.4f}  accuracy {acc:.3f}")
    return acc


if __name__ == "__main__":
    main(device="cuda" if torch.cuda.is_available() else "cpu")

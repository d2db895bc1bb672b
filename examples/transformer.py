"""Two-layer transformer encoder on a sequence parity task (the reference's
examples/transformer/main.go): predict whether a 0/1 sequence has an even number of ones."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from gonn_b200 import nn, optim  # noqa: E402


class ParityNet(nn.Module):
    def __init__(self, d=32, device="cpu"):
        super().__init__()
        self.emb = nn.Embedding(2, d, device=device)
        self.pos = nn.Embedding(8, d, device=device)
        self.enc = nn.TransformerEncoder(2, d, 4, 64, pre_norm=True, device=device)
        self.head = nn.Linear(d, 2, device=device)

    def forward(self, ids):
        pos = torch.arange(ids.shape[1], device=ids.device)
        h = self.enc(self.emb(ids) + self.pos(pos)[None])
        return self.head(h.mean(1))


def main(steps: int = 150, device: str = "cpu"):
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 2, (128, 8), generator=g).to(device)
    y = (ids.sum(1) % 2).to(device)
    model = ParityNet(device=device)
    opt = optim.AdamW(model.parameters(), lr=3e-3, weight_decay=0.0)
    first = last = None
    for step in range(steps):
        opt.zero_grad()
        loss = nn.CrossEntropyLoss(model(ids), y)
        loss.backward()
        opt.step()
        first = first if first is not None else loss.item()
        last = loss.item()
        if step % 25 == 0:
            print(f"step {step:3d}  loss {last:.4f}")
    return first, last


if __name__ == "__main__":
    main(device="cuda" if torch.cuda.is_available() else "cpu")

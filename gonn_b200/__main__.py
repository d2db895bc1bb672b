"""``python -m gonn_b200``: the entry-point demo of the reference (main.go:11-100) — basic ops,
autograd through a small expression, a matrix product and the activation registry — on the GPU
when there is one, else on the host path."""
from __future__ import annotations

import torch

from . import tensor as T


def demo_basic_ops(dev):
    print("[1] Basic ops")
    x = T.New([1, 2, 3, 4, 5, 6], 2, 3).to(dev)
    y = T.New([7, 8, 9, 10, 11, 12], 2, 3).to(dev)
    print("  x =", T.String(x))
    print("  y =", T.String(y))
    print("  x + y =", T.String(T.Add(x, y)))
    print("  x * y =", T.String(T.Mul(x, y)))
    print("  sum(x)=", T.String(T.Sum(x)))
    print()


def demo_autograd(dev):
    print("[2] Autograd: d/dx [sum((Wx)^2)] for x = [1,2,3]")
    x = T.SetRequiresGrad(T.New([1, 2, 3], 3, 1).to(dev))
    W = T.SetRequiresGrad(T.New([2, -1, 0.5], 1, 3).to(dev))
    y = T.Sum(T.Unary(T.MatMul(W, x), "square"))
    T.Backward(y)
    print("  y =", T.String(y.detach()))
    print("  dy/dx =", T.String(x.grad))
    print("  dy/dW =", T.String(W.grad))
    print()


def demo_matmul(dev):
    print("[3] MatMul (2,3) x (3,2)")
    a = T.New([1, 2, 3, 4, 5, 6], 2, 3).to(dev)
    b = T.New([1, 0, 0, 1, 1, 1], 3, 2).to(dev)
    print("  a @ b =", T.String(T.MatMul(a, b)))
    print()


def demo_activations(dev):
    print("[4] Activations from the registry")
    x = T.New([-2, -1, 0, 1, 2], 5).to(dev)
    for name in ("relu", "sigmoid", "tanh", "gelu", "silu"):
        print(f"  {name:8s}", T.String(T.Unary(x, name)))
    print(f"  {len(T.UnaryOpNames())} unary ops registered")


def main():
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    print("gonn_b200 — B200-native framework with the reference's vocabulary")
    print("=================================================================")
    print(f"device: {dev}\n")
    for demo in (demo_basic_ops, demo_autograd, demo_matmul, demo_activations):
        demo(dev)


if __name__ == "__main__":
    main()

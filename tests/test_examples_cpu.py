"""The example programs run end to end on the CPU and learn their toy tasks."""
import importlib.util
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(name):
    spec = importlib.util.spec_from_file_location(f"example_{name}", os.path.join(ROOT, "examples", f"{name}.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_regression():
    assert _load("regression").main(steps=120) < 0.02


def test_mlp():
    assert _load("mlp").main(epochs=6) > 0.9


def test_cnn():
    assert _load("cnn").main(steps=30) > 0.9


def test_transformer():
    first, last = _load("transformer").main(steps=60)
    assert last < first


def test_ml_classical():
    scores = _load("ml_classical").main()
    assert min(scores.values()) > 0.8


def test_smoke():
    _load("smoke").main()

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


def test_package_entry_point_demo(capsys):
    from gonn_b200 import __main__ as demo
    demo.main()
    out = capsys.readouterr().out
    assert "x + y = Tensor(shape=[2 3], data=[8 10 12 14 16 18])" in out
    assert "dy/dx = Tensor(shape=[3 1], data=[6 -3 1.5])" in out and "dy/dW = Tensor(shape=[1 3], data=[3 6 9])" in out
    assert "a @ b = Tensor(shape=[2 2], data=[4 5 10 11])" in out and "unary ops registered" in out


def test_reference_style_program():
    assert _load("reference_style").main(epochs=60, verbose=False) > 0.95

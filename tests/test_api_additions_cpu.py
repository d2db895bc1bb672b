"""Small API pieces that need no GPU: activation kinds from the registry, exported constructor names,
upsampling aliases, the flags of the cross-entropy and attention-backward paths, the debug-build
selection, and the command line of the benchmark."""
import json
import os
import subprocess
import sys

import pytest
import torch

from gonn_b200 import nn, tensor as T

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_activation_accepts_registered_and_rejects_unknown_names():
    from gonn_b200.tensor import api
    saved = dict(api._REGISTRY)
    try:
        T.RegisterUnary(T.UnaryOpDef("cube_demo", lambda x: x ** 3, lambda x, g: 3 * g * x ** 2))
        act = nn.Activation("cube_demo")
        x = torch.tensor([1.0, -2.0], dtype=torch.float64, requires_grad=True)
        act(x).sum().backward()
        assert torch.equal(x.grad, torch.tensor([3.0, 12.0], dtype=torch.float64))
        with pytest.raises(KeyError):
            nn.Activation("no_such_op")
        assert float(nn.Activation("relu")(torch.tensor([-1.0]))) == 0.0
    finally:
        api._REGISTRY.clear()
        api._REGISTRY.update(saved)


def test_sync_batchnorm_constructors_are_exported_lazily():
    from gonn_b200 import distributed
    for name in ("SyncBatchNorm1d", "SyncBatchNorm2d", "SyncBatchNorm3d", "NewSyncBatchNorm1d",
                 "NewSyncBatchNorm2d", "NewSyncBatchNorm3d", "convert_sync_batchnorm", "DistributedDataParallel"):
        assert callable(getattr(distributed, name)), name
    with pytest.raises(AttributeError):
        distributed.NoSuchThing


@pytest.mark.parametrize("alias,mode,kw", [("UpsamplingNearest2d", "nearest", {}),
                                           ("UpsamplingBilinear2d", "bilinear", {"align_corners": True})])
def test_upsampling_aliases_match_torch(alias, mode, kw):
    x = torch.randn(2, 3, 5, 4, dtype=torch.float64)
    got = getattr(nn, alias)(2)(x)
    want = torch.nn.functional.interpolate(x, scale_factor=2, mode=mode, **kw)
    torch.testing.assert_close(got, want, rtol=1e-12, atol=1e-12)


def test_consume_logits_is_ignored_on_the_host_path():
    from gonn_b200.ops.softmax import cross_entropy
    x = torch.randn(9, 16, dtype=torch.float32, requires_grad=True)
    t = torch.randint(0, 16, (9,))
    keep = x.detach().clone()
    loss = cross_entropy(x, t, inplace_backward=True, consume_logits=True)
    loss.backward()
    assert torch.equal(x.detach(), keep)                          # nothing was overwritten
    xr = keep.clone().requires_grad_(True)
    torch.nn.functional.cross_entropy(xr, t).backward()
    torch.testing.assert_close(x.grad, xr.grad, rtol=1e-5, atol=1e-6)


def test_ds_spill_limit_is_capped_at_what_the_kernel_can_address():
    from gonn_b200.ops import attention as A
    old = A.DS_SPILL_LIMIT_BYTES
    try:
        A.set_ds_spill_limit(1 << 40)
        assert A.DS_SPILL_LIMIT_BYTES == 1 << 32
        A.set_ds_spill_limit(0)
        assert A._ds_workspace(torch.device("cpu"), 1024) is None
    finally:
        A.set_ds_spill_limit(old)


def test_debug_build_recompiles_only_units_with_checks():
    from gonn_b200 import build
    checked = sorted(n for n in build._sources() if build._has_checks(n))
    assert checked == ["embedding.cu", "norm.cu", "reduce.cu", "runtime.cu", "window.cu"]
    assert build.DEBUG_LIB.endswith("libgonn_b200_debug.so") and build.LIB.endswith("libgonn_b200.so")


def test_library_relinks_when_an_object_is_newer(tmp_path, monkeypatch):
    """The two libraries share most objects: an object rebuilt by one flavour's pass must relink the
    other library too, although that pass compiled nothing."""
    from gonn_b200 import build
    obj_dir = tmp_path / "obj"
    obj_dir.mkdir()
    lib = tmp_path / "lib.so"
    lib.write_bytes(b"")
    monkeypatch.setattr(build, "OBJ_DIR", str(obj_dir))
    monkeypatch.setattr(build, "LIB", str(lib))
    monkeypatch.setattr(build, "_sources", lambda: ["a.cu", "b.cu"])
    monkeypatch.setattr(build, "_compile", lambda n, v, f, d=False: (n, False, ""))
    past = os.path.getmtime(lib) - 100
    for n in ("a.o", "b.o"):
        (obj_dir / n).write_bytes(b"")
        os.utime(obj_dir / n, (past, past))
    links = []

    class Done:
        returncode, stdout, stderr = 0, "", ""

    monkeypatch.setattr(build.subprocess, "run", lambda cmd, **kw: links.append(cmd) or Done())
    build.build()
    assert links == []                                    # nothing compiled, nothing newer: no link
    future = os.path.getmtime(lib) + 100
    os.utime(obj_dir / "b.o", (future, future))
    build.build()
    assert len(links) == 1 and "-shared" in links[0] and str(obj_dir / "b.o") in links[0]


def test_library_path_follows_the_environment():
    code = "import gonn_b200.lib as L; print(L.LIB_PATH); print(L.DEBUG_BUILD)"
    env = dict(os.environ, PYTHONPATH=ROOT)
    env.pop("GONN_B200_LIB", None)
    out = subprocess.run([sys.executable, "-c", code], env=dict(env, GONN_B200_DEBUG="1"), capture_output=True, text=True)
    assert "libgonn_b200_debug.so" in out.stdout and "True" in out.stdout
    out = subprocess.run([sys.executable, "-c", code], env=dict(env, GONN_B200_LIB="/tmp/other.so"), capture_output=True, text=True)
    assert out.stdout.splitlines()[0] == "/tmp/other.so"


def test_benchmark_reference_arm_answers_without_a_gpu():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference"], capture_output=True,
                         text=True, cwd=ROOT, timeout=300)
    assert out.returncode == 0
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line
    assert len(out.stdout.strip().splitlines()) == 1
    other = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2"],
                           capture_output=True, text=True, cwd=ROOT, timeout=300, env=dict(os.environ, RANK="1"))
    assert other.returncode == 0 and other.stdout.strip() == ""      # one line per job: only rank 0 prints
    help_text = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--help"], capture_output=True,
                               text=True, cwd=ROOT, timeout=300).stdout
    for flag in ("--gpus", "--steps", "--warmup", "--impl", "--config", "--no-graph", "--no-overlap", "--quick"):
        assert flag in help_text


def test_mha_benchmark_runs_on_the_cpu_path(capsys):
    """The reference's Forward / ForwardFused benchmark (small size here): both entry points agree and
    one JSON line comes out."""
    from gonn_b200.utils import microbench
    rec = microbench.bench_mha("cpu", B=2, S=32, E=32, H=2, iters=2)
    assert rec["diffs"][False] < 1e-12 and rec["diffs"][True] < 1e-12
    assert rec["forward_ms"] > 0 and rec["forward_fused_ms"] > 0
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert line["bench"] == "mha" and line["device"] == "cpu" and line["causal"] is True

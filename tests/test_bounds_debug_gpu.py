"""The bounds-checked build (``python -m gonn_b200.build --debug``), run in a child process with
``GONN_B200_DEBUG=1`` so that this process keeps the regular library.

Two things are checked.  Correct programs stay silent: pooling, embedding, normalisation and
reductions produce the same results as the regular build and leave the status word clear.  And a
table entry that points outside its buffer is reported, not followed: the child hands the pooling
kernel an index map whose last entry is one past the plane; the checked kernel records status 7
(out of bounds) with the site number and skips the load, the context stays usable, and the next
operation gives the right answer.  The child refuses to run that part unless the loaded library
says it is the checked build.
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

CHILD = r"""
import numpy as np, torch
from gonn_b200 import lib as L, nn
from gonn_b200.ops import window as win
from gonn_b200.ops.norm import layer_norm
from gonn_b200.ops.reduce import column_sum
lib = L.lib()
assert lib.gb_bounds_checked_build() == 1, "not the bounds-checked library"
dev = "cuda"
# 1. correct programs: same answers, clear status word
x = torch.randn(8, 16, 14, 14, device=dev, dtype=torch.bfloat16, requires_grad=True)
y = nn.MaxPool2d(2)(x); y.sum().backward()
assert torch.equal(y.float(), torch.nn.functional.max_pool2d(x.detach().float(), 2))
a = nn.AvgPool2d(3, 2, 1)(x.detach())
assert (a.float() - torch.nn.functional.avg_pool2d(x.detach().float(), 3, 2, 1)).abs().max() < 2e-2
emb = nn.Embedding(1000, 72, dtype=torch.bfloat16, device=dev)
ids = torch.randint(0, 1000, (4, 333), device=dev)
emb(ids).sum().backward()
ref = torch.zeros(1000, 72, device=dev).index_add_(0, ids.view(-1), torch.ones(ids.numel(), 72, device=dev))
assert (emb.weight.grad.float() - ref).abs().max() < 1e-2 * ref.max()
h = torch.randn(4099, 768, device=dev, dtype=torch.bfloat16, requires_grad=True)
w = torch.ones(768, device=dev, dtype=torch.bfloat16, requires_grad=True)
b = torch.zeros(768, device=dev, dtype=torch.bfloat16, requires_grad=True)
layer_norm(h, w, b).sum().backward()
assert (column_sum(h.detach()).float() - h.detach().float().sum(0)).abs().max() < 2.0
L.assert_status_ok()
# 2. an index map entry one past the plane: reported through the status word, access skipped
H = W = 6; S = H * W; B = 4
idx_np, _ = win.sliding_index((H, W), 2, 2, 0, 1)
bad = idx_np.copy(); bad[-1, -1] = S                       # valid entries are 0 .. S-1
xx = torch.zeros(B * S + 64, device=dev, dtype=torch.float32)[:B * S].view(B, S)   # slack behind the plane
idx_dev = torch.from_numpy(bad).to(dev)
nwin, T = bad.shape
yy = torch.empty(B, nwin, device=dev); arg = torch.empty(B, nwin, device=dev, dtype=torch.int32)
L.call("gb_pool_fwd", L.I(2), L.ptr(xx), L.ptr(idx_dev), L.ptr(yy), L.ptr(arg), L.L(B), L.L(S), L.I(nwin), L.I(T),
       L.I(0), L.I(0), L.F(2.0), L.stream_ptr())
code, detail, block, count = L.read_status()
assert code == 7 and detail == 103 and count == B, (code, detail, block, count)
# the context is intact and the word was cleared by the read
z = nn.MaxPool2d(2)(x.detach())
assert torch.equal(z.float(), torch.nn.functional.max_pool2d(x.detach().float(), 2))
L.assert_status_ok()
print("BOUNDS-OK")
"""


def test_bounds_checked_build_reports_and_skips_out_of_range_indices():
    from gonn_b200 import build
    if not os.path.exists(build.DEBUG_LIB):
        build.build(debug=True)
    env = dict(os.environ, GONN_B200_DEBUG="1")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env["PYTHONPATH"] = root + os.pathsep + env.get("PYTHONPATH", "")
    r = subprocess.run([sys.executable, "-c", CHILD], env=env, capture_output=True, text=True, timeout=600, cwd=root)
    assert r.returncode == 0 and "BOUNDS-OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]

"""The canary-padded buffer helper itself, on the host: a byte changed outside the tensor is found
and attributed to the right side."""
import pytest
import torch

from gonn_b200.utils.canary import PATTERN, guarded


def test_guard_zones_detect_a_stray_store_on_the_host_side():
    g = guarded((5, 7), torch.float32, device="cpu", fill=0.0)
    g.check()
    g.raw[g._hi + 3] = 0          # what a kernel writing one element too far would do
    with pytest.raises(AssertionError, match="after the tensor"):
        g.check()
    g.raw[g._hi + 3] = PATTERN
    g.raw[g._lo - 1] = 1
    with pytest.raises(AssertionError, match="before the tensor"):
        g.check()


def test_misaligned_payload_keeps_its_guards():
    g = guarded((3, 5), torch.bfloat16, device="cpu", fill=1.0, misalign=2)
    assert g.t.data_ptr() % 16 == 2 or g.t.data_ptr() % 4 == 2
    g.check()
    assert float(g.t.float().sum()) == 15.0

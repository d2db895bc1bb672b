"""Property tests (hypothesis) of the host-side logic the kernels rely on: window index maps and
their CSR inverse, the data-parallel bucket layout (alignment rules of the vector and TMA
accesses), and shard bounds."""
import numpy as np
import torch
import torch.nn.functional as F
from hypothesis import given, settings, strategies as st

from gonn_b200.ops import window as W
from gonn_b200.parallel.data_parallel import shard_bounds

_cfg = settings(max_examples=60, deadline=None)


@_cfg
@given(h=st.integers(3, 9), w=st.integers(3, 9), k=st.integers(1, 3), s=st.integers(1, 3), p=st.integers(0, 2),
       d=st.integers(1, 2))
def test_sliding_index_reproduces_unfold(h, w, k, s, p, d):
    if (k - 1) * d + 1 > min(h, w) + 2 * p or p > k // 2 + 1:
        return
    idx, outs = W.sliding_index((h, w), k, s, p, d)
    x = torch.arange(1, h * w + 1, dtype=torch.float64).reshape(1, 1, h, w)
    ref = F.unfold(x, k, dilation=d, padding=p, stride=s)[0].t()          # (nwin, k*k)
    flat = torch.cat([x.reshape(-1), torch.zeros(1, dtype=torch.float64)])  # index -1 reads the zero
    got = flat[torch.from_numpy(idx.astype(np.int64))]
    assert idx.shape == (outs[0] * outs[1], k * k) and torch.equal(got, ref)
    assert idx.max() < h * w and idx.min() >= -1


@_cfg
@given(h=st.integers(2, 7), w=st.integers(2, 7), k=st.integers(1, 3), s=st.integers(1, 2), p=st.integers(0, 1))
def test_csr_inverse_lists_every_tap_once(h, w, k, s, p):
    if k > min(h, w) + 2 * p:
        return
    idx, _ = W.sliding_index((h, w), k, s, p, 1)
    S = h * w
    key = (idx.shape, hash(idx.tobytes()), S)
    W._MAPS.setdefault(key, idx)
    offs, cols = W._invert_cached(key, S)
    flat = idx.reshape(-1)
    assert offs[0] == 0 and offs[-1] == (flat >= 0).sum() == len(cols) and (np.diff(offs) >= 0).all()
    for pos in range(S):
        taps = cols[offs[pos]:offs[pos + 1]]
        assert (flat[taps] == pos).all() and len(set(taps.tolist())) == len(taps)
    assert sorted(cols.tolist()) == np.nonzero(flat >= 0)[0].tolist()


@_cfg
@given(sizes=st.lists(st.integers(1, 700), min_size=1, max_size=12), world=st.sampled_from([1, 2, 4, 8]),
       bucket_elems=st.integers(1, 900))
def test_bucket_layout_alignment(sizes, world, bucket_elems):
    """Every parameter starts on an 8-element (16-byte) boundary inside its bucket, buckets tile
    the buffer without gaps or overlap, and every bucket divides into ``world`` shards of whole
    16-byte vectors."""
    from gonn_b200.distributed.ddp import plan_buckets
    offsets, buckets, total = plan_buckets(sizes, world, bucket_elems)
    assert len(offsets) == len(sizes) and sorted(i for _, _, m in buckets for i in m) == list(range(len(sizes)))
    pos = 0
    for start, length, members in buckets:
        assert start == pos and length > 0 and length % (world * 8) == 0 and (length // world) % 8 == 0
        pos += length
        for i in members:
            assert offsets[i] % 8 == 0 and start <= offsets[i] and offsets[i] + sizes[i] <= start + length
    assert pos == total
    for i in range(len(sizes) - 1):                        # packed in order, no overlap
        assert offsets[i] + sizes[i] <= offsets[i + 1]
    # all but the last bucket reached the size limit
    assert all(length >= min(max(bucket_elems, world * 8), length) for _, length, _ in buckets[:-1])


def test_engine_uses_the_planned_layout():
    from gonn_b200.distributed.ddp import DistributedDataParallel, plan_buckets
    sizes = [5, 300, 17, 64, 1000, 3]

    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.ps = torch.nn.ParameterList([torch.nn.Parameter(torch.zeros(n, dtype=torch.bfloat16)) for n in sizes])

    eng = DistributedDataParallel(M(), optimizer=None, bucket_mb=256 * 2 / (1 << 20), rank=0, world=1)
    offsets, buckets, total = plan_buckets(sizes, 1, 256)
    assert [(b.start, b.length) for b in eng.buckets] == [(s, l) for s, l, _ in buckets] and eng.total == total
    assert [eng._where[id(p)][1] for p in eng.params] == offsets
    for p in eng.params:                                   # parameters and gradients live in the flat buffers
        _, o, n = eng._where[id(p)]
        assert p.data_ptr() == eng.flat_params[o:o + n].data_ptr() and p.grad.data_ptr() == eng.flat_grads[o:o + n].data_ptr()


@_cfg
@given(n=st.integers(1, 200), workers=st.integers(1, 16))
def test_shard_bounds_cover_the_batch(n, workers):
    b = shard_bounds(n, workers)
    assert b[0][0] == 0 and b[-1][1] == n and all(lo < hi for lo, hi in b)
    assert all(b[i][1] == b[i + 1][0] for i in range(len(b) - 1))
    sizes = [hi - lo for lo, hi in b]
    assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True) and len(b) == min(workers, n)

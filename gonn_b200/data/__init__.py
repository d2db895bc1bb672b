"""Datasets, the batching loader, transforms and synthetic generators (data/*.go).

``Dataset`` = ``Len()`` / ``Get(i) -> (x, y)``; ``TensorDataset`` deep-copies rows on ``Get``;
``DataLoader`` batches with optional seeded shuffling and drop-last, collating with ``stack``;
with ``pin_memory`` / ``device`` it stages batches in pinned host memory and copies them to
the device on a side stream one batch ahead.
"""
from __future__ import annotations

import csv
import gzip
import os
import struct
import threading
import queue
from typing import Callable, Iterator, List, NamedTuple, Optional, Sequence, Tuple

import numpy as np
import torch


class Dataset:
    def Len(self) -> int:
        raise NotImplementedError

    def Get(self, i: int):
        raise NotImplementedError

    def __len__(self):
        return self.Len()

    def __getitem__(self, i):
        return self.Get(i)


class TensorDataset(Dataset):
    def __init__(self, X: torch.Tensor, Y: torch.Tensor):
        if X.shape[0] != Y.shape[0]:
            raise ValueError("TensorDataset: X and Y must have the same number of rows")
        self.X, self.Y = X, Y

    def Len(self):
        return self.X.shape[0]

    def Get(self, i):
        return self.X[i].clone(), self.Y[i].clone()


class Subset(Dataset):
    def __init__(self, base: Dataset, indices: Sequence[int]):
        self.base, self.indices = base, list(indices)

    def Len(self):
        return len(self.indices)

    def Get(self, i):
        return self.base.Get(self.indices[i])


class ConcatDataset(Dataset):
    def __init__(self, *parts: Dataset):
        self.parts = list(parts)
        self.offsets = np.cumsum([0] + [p.Len() for p in self.parts])

    def Len(self):
        return int(self.offsets[-1])

    def Get(self, i):
        if not 0 <= i < self.Len():
            raise IndexError(i)
        k = int(np.searchsorted(self.offsets, i, side="right") - 1)
        return self.parts[k].Get(i - int(self.offsets[k]))


class Batch(NamedTuple):
    """One mini-batch (data/dataloader.go:11-14); unpacks as ``x, y``."""
    X: torch.Tensor
    Y: torch.Tensor


class DataLoader:
    def __init__(self, dataset: Dataset, batch_size: int = 1, shuffle: bool = False, drop_last: bool = False,
                 seed: int = 0, transform: Optional[Callable] = None, device=None, pin_memory: bool = False,
                 prefetch: int = 2):
        self.dataset, self.BatchSize, self.Shuffle, self.DropLast, self.Seed = dataset, batch_size, shuffle, drop_last, seed
        self.transform, self.device, self.pin_memory, self.prefetch = transform, device, pin_memory, prefetch
        self._epoch = 0

    def __len__(self):
        n = self.dataset.Len()
        return n // self.BatchSize if self.DropLast else -(-n // self.BatchSize)

    Len = __len__           # number of batches per epoch (data/dataloader.go)
    Dataset = property(lambda self: self.dataset)

    def _batches(self):
        n = self.dataset.Len()
        order = np.arange(n)
        if self.Shuffle:
            order = np.random.default_rng(self.Seed + self._epoch).permutation(n)
        self._epoch += 1
        for s in range(0, n, self.BatchSize):
            idx = order[s:s + self.BatchSize]
            if len(idx) < self.BatchSize and self.DropLast:
                return
            xs, ys = zip(*(self.dataset.Get(int(i)) for i in idx))
            if self.transform is not None:
                xs = [self.transform(x) for x in xs]
            yield Batch(torch.stack(list(xs)), torch.stack(list(ys)))

    def Iter(self) -> Iterator[Tuple[torch.Tensor, torch.Tensor]]:
        """Batches produced by a background thread (the reference feeds a channel from a goroutine)."""
        q: "queue.Queue" = queue.Queue(maxsize=max(self.prefetch, 1))
        stop = object()
        to_dev = self.device is not None and torch.device(self.device).type == "cuda"

        def work():
            try:
                for x, y in self._batches():
                    if self.pin_memory or to_dev:
                        x, y = x.pin_memory(), y.pin_memory()
                    q.put((x, y))
            finally:
                q.put(stop)

        t = threading.Thread(target=work, daemon=True)
        t.start()
        copy_stream = torch.cuda.Stream() if to_dev else None
        while True:
            item = q.get()
            if item is stop:
                break
            x, y = item
            if to_dev:
                with torch.cuda.stream(copy_stream):
                    xd, yd = x.to(self.device, non_blocking=True), y.to(self.device, non_blocking=True)
                torch.cuda.current_stream().wait_stream(copy_stream)
                yield Batch(xd, yd)
            else:
                yield Batch(x, y)

    __iter__ = Iter


# ---- transforms (data/transforms.go:13-180) --------------------------------------------------
class Transform:
    """A per-sample transform: ``Apply(t) -> tensor`` (data/transforms.go:13-15); instances are
    also callable, which is how the ``DataLoader`` uses them."""

    def Apply(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def __call__(self, x):
        return self.Apply(x)


class Normalize(Transform):
    """Per leading channel: (x - mean[c]) / std[c]; the lengths must match the channel count and
    no std may be zero (data/transforms.go:28-49)."""

    def __init__(self, mean: Sequence[float], std: Sequence[float]):
        self.Mean, self.Std = list(mean), list(std)

    def Apply(self, x):
        if x.dim() == 0:
            raise ValueError("data.Normalize: cannot normalize a 0-D tensor")
        c = x.shape[0]
        if len(self.Mean) != c or len(self.Std) != c:
            raise ValueError(f"data.Normalize: mean/std length {len(self.Mean)}/{len(self.Std)} must match "
                             f"channel dim {c}")
        if any(v == 0 for v in self.Std):
            raise ValueError("data.Normalize: std has a zero entry")
        shape = [-1] + [1] * (x.dim() - 1)
        dt = x.dtype if x.is_floating_point() else torch.float32
        mean = torch.tensor(self.Mean, dtype=dt, device=x.device).reshape(shape)
        std = torch.tensor(self.Std, dtype=dt, device=x.device).reshape(shape)
        return (x.to(dt) - mean) / std


class RandomHorizontalFlip(Transform):
    """Flips the last dimension with probability ``P`` (0 or less: never)."""

    def __init__(self, p: float = 0.5, seed: Optional[int] = None):
        self.P, self.Rand = p, np.random.default_rng(seed)

    def Apply(self, x):
        if self.P <= 0:
            return x.clone()
        return x.flip(-1) if self.Rand.random() < self.P else x.clone()


class RandomCrop(Transform):
    """Crops the trailing ``len(size)`` dimensions to ``size`` at a uniformly drawn offset; an
    integer crops the last two dimensions to a square (data/transforms.go:103-150)."""

    def __init__(self, size, seed: Optional[int] = None):
        self.Size = [size, size] if isinstance(size, int) else list(size)
        self.Rand = np.random.default_rng(seed)

    def Apply(self, x):
        if not self.Size:
            return x.clone()
        if len(self.Size) > x.dim():
            raise ValueError(f"data.RandomCrop: size {self.Size} has more dims than tensor shape {list(x.shape)}")
        off = x.dim() - len(self.Size)
        sl = [slice(None)] * x.dim()
        for i, s in enumerate(self.Size):
            dim = x.shape[off + i]
            if s > dim or s <= 0:
                raise ValueError(f"data.RandomCrop: crop size {s} invalid for dim {off + i} (size {dim})")
            o = int(self.Rand.integers(0, dim - s + 1)) if dim > s else 0
            sl[off + i] = slice(o, o + s)
        return x[tuple(sl)].clone()


class ToFloat(Transform):
    """Converts to floating point.  The reference's tensors are always float64, so there it is
    the identity (data/transforms.go:160-162); here integer images become float32, optionally
    scaled (``scale=1/255`` maps bytes to [0, 1])."""

    def __init__(self, scale: float = 1.0):
        self.scale = scale

    def Apply(self, x):
        y = x if x.is_floating_point() else x.to(torch.float32)
        return y * self.scale if self.scale != 1.0 else y


class Compose(Transform):
    def __init__(self, *ts):
        if len(ts) == 1 and isinstance(ts[0], (list, tuple)):
            ts = tuple(ts[0])
        self.Transforms = list(ts)

    def Apply(self, x):
        for t in self.Transforms:
            x = t(x)
        return x


def _read_idx(path):
    opener = gzip.open if path.endswith(".gz") else open
    with opener(path, "rb") as f:
        raw = f.read()
    magic, = struct.unpack(">I", raw[:4])
    nd = magic & 0xFF
    dims = struct.unpack(">" + "I" * nd, raw[4:4 + 4 * nd])
    return np.frombuffer(raw, dtype=np.uint8, offset=4 + 4 * nd).reshape(dims)


def LoadMNIST(directory: str):
    """Reads the four IDX files (raw or .gz) from ``directory``; never downloads.  Returns
    (train TensorDataset (60000,1,28,28), test TensorDataset (10000,1,28,28)), pixels in [0,1]."""
    def find(stem):
        for cand in (stem, stem + ".gz"):
            p = os.path.join(directory, cand)
            if os.path.exists(p):
                return p
        raise FileNotFoundError(f"LoadMNIST: {stem}[.gz] not found in {directory}")
    out = []
    for img, lab in (("train-images-idx3-ubyte", "train-labels-idx1-ubyte"),
                     ("t10k-images-idx3-ubyte", "t10k-labels-idx1-ubyte")):
        X = torch.from_numpy(_read_idx(find(img)).astype(np.float32) / 255.0)[:, None]
        Y = torch.from_numpy(_read_idx(find(lab)).astype(np.int64))
        out.append(TensorDataset(X, Y))
    return tuple(out)


def LoadCSV(path: str, has_header: bool = True, target_col: int = -1, dtype=torch.float64):
    """Numeric CSV -> TensorDataset; a negative ``target_col`` counts from the end."""
    with open(path, newline="") as f:
        rows = list(csv.reader(f))
    if has_header:
        rows = rows[1:]
    arr = np.asarray([[float(v) for v in r] for r in rows if r], dtype=np.float64)
    tc = target_col % arr.shape[1]
    X = np.delete(arr, tc, axis=1)
    return TensorDataset(torch.from_numpy(X).to(dtype), torch.from_numpy(arr[:, tc].copy()).to(dtype))


# ---- synthetic generators (data/synthetic.go:10-170) ---------------------------------------------
class _XY(tuple):
    """``(X, y)`` as the reference returns it (data/synthetic.go:16), with the generating
    coefficients of a regression problem kept in ``Weights``."""
    Weights = None


def MakeRegression(n: int, d: int, noise: float = 0.1, seed: int = 0):
    """``X, y = MakeRegression(n, d, noise, seed)``; the true coefficients are ``.Weights`` of
    the returned pair."""
    r = np.random.default_rng(seed)
    X = r.standard_normal((n, d))
    w = r.standard_normal(d)
    y = X @ w + noise * r.standard_normal(n)
    out = _XY((torch.from_numpy(X), torch.from_numpy(y)))
    out.Weights = torch.from_numpy(w)
    return out


def MakeBlobs(n: int, d: int, centers: int, seed: int = 0, *, std: float = 1.0):
    r = np.random.default_rng(seed)
    C = r.uniform(-10, 10, (centers, d))
    y = r.integers(0, centers, n)
    X = C[y] + std * r.standard_normal((n, d))
    return torch.from_numpy(X), torch.from_numpy(y.astype(np.int64))


def MakeClassification(n: int, d: int, classes: int = 2, seed: int = 0, *, sep: float = 3.0):
    r = np.random.default_rng(seed)
    C = r.standard_normal((classes, d)) * sep
    y = r.integers(0, classes, n)
    X = C[y] + r.standard_normal((n, d))
    return torch.from_numpy(X), torch.from_numpy(y.astype(np.int64))


def MakeMoons(n: int, noise: float = 0.1, seed: int = 0):
    r = np.random.default_rng(seed)
    n0 = n // 2
    t0, t1 = np.linspace(0, np.pi, n0), np.linspace(0, np.pi, n - n0)
    X = np.concatenate([np.stack([np.cos(t0), np.sin(t0)], 1), np.stack([1 - np.cos(t1), 0.5 - np.sin(t1)], 1)])
    X += noise * r.standard_normal(X.shape)
    y = np.concatenate([np.zeros(n0), np.ones(n - n0)]).astype(np.int64)
    return torch.from_numpy(X), torch.from_numpy(y)


def _constructor_aliases(ns) -> None:
    """``NewX`` for every public class ``X`` (the reference's constructor functions)."""
    for name, obj in list(ns.items()):
        if isinstance(obj, type) and name[0].isupper() and "New" + name not in ns:
            ns["New" + name] = _accepting_options(obj)


from ..options import accepting_options as _accepting_options, package_getattr as _package_getattr  # noqa: E402

_constructor_aliases(globals())
__getattr__ = _package_getattr(__name__)     # optim.WithMomentum(0.9), optim.WithNesterov(True), ...

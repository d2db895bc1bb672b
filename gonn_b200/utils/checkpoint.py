"""Checkpoint format: save / load of module parameters, buffers and optimizer state.

The reference has no serializer; it fixes the ingredients a checkpoint needs: dotted
parameter names and registration order (nn/module.go:103-128), buffer names
(nn/batchnorm.go:35-36), frozen optimizer-state buffer names (optim/state.go:3-17) and one
on-the-wire number encoding, big-endian IEEE-754 float64 (distributed/distributed.go:18-24).
The container below is built from exactly those pieces:

    magic "GONNCKPT" | u32 version | u32 entry count | entries...
    entry: u16 name length | name (utf-8) | u8 kind | u8 dtype | u8 rank | u64 dims... | payload

``kind``: 0 parameter, 1 buffer, 2 optimizer buffer, 3 scalar.  ``dtype`` selects the payload
encoding: 0 = big-endian float64 (the reference's wire encoding, exact for fp64 models),
1 = big-endian float32, 2 = bf16 (big-endian 16-bit), 3 = big-endian int64.  Entries appear
as ``NamedParameters()`` then ``Buffers()`` then optimizer state ``<param name>/<buffer>``
and scalars ``<param name>/@<scalar>`` / ``@opt/<scalar>``.
"""
from __future__ import annotations

import struct
from typing import Dict, Optional

import numpy as np
import torch

MAGIC = b"GONNCKPT"
VERSION = 1
_K_PARAM, _K_BUF, _K_OPT, _K_SCALAR = 0, 1, 2, 3
_DT = {torch.float64: 0, torch.float32: 1, torch.bfloat16: 2, torch.int64: 3}
_DT_INV = {v: k for k, v in _DT.items()}


def _encode(t: torch.Tensor, dtype_code: int) -> bytes:
    t = t.detach().cpu().contiguous()
    if dtype_code == 0:
        return t.to(torch.float64).numpy().astype(">f8").tobytes()
    if dtype_code == 1:
        return t.to(torch.float32).numpy().astype(">f4").tobytes()
    if dtype_code == 2:
        return t.to(torch.bfloat16).view(torch.int16).numpy().astype(">i2").tobytes()
    return t.to(torch.int64).numpy().astype(">i8").tobytes()


def _decode(raw: bytes, dtype_code: int, shape) -> torch.Tensor:
    if dtype_code == 0:
        a = np.frombuffer(raw, dtype=">f8").astype(np.float64)
        return torch.from_numpy(a).reshape(shape)
    if dtype_code == 1:
        return torch.from_numpy(np.frombuffer(raw, dtype=">f4").astype(np.float32)).reshape(shape)
    if dtype_code == 2:
        a = np.frombuffer(raw, dtype=">i2").astype(np.int16)
        return torch.from_numpy(a).view(torch.bfloat16).reshape(shape)
    return torch.from_numpy(np.frombuffer(raw, dtype=">i8").astype(np.int64)).reshape(shape)


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype in _DT:
        return _DT[t.dtype]
    if t.dtype == torch.float16:
        return 1
    if not t.dtype.is_floating_point:
        return 3
    return 0


def _write_entry(f, name: str, kind: int, t: torch.Tensor):
    code = _dtype_code(t)
    nb = name.encode()
    f.write(struct.pack(">H", len(nb)) + nb + struct.pack(">BBB", kind, code, t.dim()))
    for d in t.shape:
        f.write(struct.pack(">Q", d))
    f.write(_encode(t, code))


def save(path: str, module: torch.nn.Module, optimizer=None) -> None:
    entries = []
    for n, p in module.named_parameters():
        entries.append((n, _K_PARAM, p.data))
    for n, b in module.named_buffers():
        entries.append((n, _K_BUF, b))
    if optimizer is not None:
        names = {id(p): n for n, p in module.named_parameters()}
        sd = optimizer.state_dict(names)
        for key, st in sd["state"].items():
            for bn, bt in st["bufs"].items():
                entries.append((f"{key}/{bn}", _K_OPT, bt))
            for sn, sv in st["scalars"].items():
                entries.append((f"{key}/@{sn}", _K_SCALAR, torch.tensor(float(sv), dtype=torch.float64)))
        for sn, sv in sd["scalars"].items():
            entries.append((f"@opt/{sn}", _K_SCALAR, torch.tensor(float(sv), dtype=torch.float64)))
        for gi, g in enumerate(sd["groups"]):
            entries.append((f"@group{gi}/lr", _K_SCALAR, torch.tensor(float(g["lr"]), dtype=torch.float64)))
            entries.append((f"@group{gi}/weight_decay", _K_SCALAR, torch.tensor(float(g["weight_decay"]), dtype=torch.float64)))
    with open(path, "wb") as f:
        f.write(MAGIC + struct.pack(">II", VERSION, len(entries)))
        for n, k, t in entries:
            _write_entry(f, n, k, t)


def read(path: str) -> Dict[str, tuple]:
    """name -> (kind, tensor), in file order."""
    out: Dict[str, tuple] = {}
    with open(path, "rb") as f:
        if f.read(8) != MAGIC:
            raise ValueError("not a checkpoint of this format (bad magic)")
        version, count = struct.unpack(">II", f.read(8))
        if version != VERSION:
            raise ValueError(f"unsupported checkpoint version {version}")
        for _ in range(count):
            (ln,) = struct.unpack(">H", f.read(2))
            name = f.read(ln).decode()
            kind, code, rank = struct.unpack(">BBB", f.read(3))
            shape = [struct.unpack(">Q", f.read(8))[0] for _ in range(rank)]
            n = int(np.prod(shape)) if shape else 1
            width = {0: 8, 1: 4, 2: 2, 3: 8}[code]
            out[name] = (kind, _decode(f.read(n * width), code, shape))
    return out


def load(path: str, module: torch.nn.Module, optimizer=None, strict: bool = True) -> None:
    """Loads values by name; tensors are converted to the destination dtype (cross-dtype loads
    such as an fp64 checkpoint into a bf16 model are allowed)."""
    ent = read(path)
    named = dict(module.named_parameters())
    named.update(dict(module.named_buffers()))
    missing = [n for n in named if n not in ent]
    if strict and missing:
        raise KeyError(f"checkpoint is missing {missing}")
    with torch.no_grad():
        for n, t in named.items():
            if n in ent:
                src = ent[n][1]
                if tuple(src.shape) != tuple(t.shape):
                    raise ValueError(f"shape mismatch for {n}: {tuple(src.shape)} vs {tuple(t.shape)}")
                t.copy_(src.to(dtype=t.dtype, device=t.device))
    if optimizer is not None:
        names = {id(p): n for n, p in module.named_parameters()}
        sd = {"groups": [], "scalars": {}, "state": {}}
        for gi, g in enumerate(optimizer.groups):
            sd["groups"].append({"lr": float(ent.get(f"@group{gi}/lr", (0, torch.tensor(g.lr)))[1]),
                                 "weight_decay": float(ent.get(f"@group{gi}/weight_decay", (0, torch.tensor(g.weight_decay)))[1]),
                                 "n": len(g.params)})
        for key, (kind, t) in ent.items():
            if kind == _K_OPT:
                pn, bn = key.rsplit("/", 1)
                sd["state"].setdefault(pn, {"bufs": {}, "scalars": {}})["bufs"][bn] = t
            elif kind == _K_SCALAR and key.startswith("@opt/"):
                sd["scalars"][key[5:]] = float(t)
            elif kind == _K_SCALAR and "/@" in key:
                pn, sn = key.rsplit("/@", 1)
                sd["state"].setdefault(pn, {"bufs": {}, "scalars": {}})["scalars"][sn] = float(t)
        optimizer.load_state_dict(sd, names)

"""safetensors reader/writer (own implementation, no third-party package).

Format: 8-byte little-endian header length, a JSON header mapping tensor name to
``{"dtype", "shape", "data_offsets"}``, then the raw little-endian tensor bytes.  Supported dtypes
are the ones the reference writes — ``U32, U64, BF16, F16, F32`` (reference:
``tensorlib/src/safe_tensors.cpp:34-76, 86-530``) — plus ``I32``/``I64`` for convenience.
``load(path, pinned=True)`` reads into page-locked memory; ``load_inplace`` fills existing tensors
after checking dtype and shape.  The native runtime (``csrc/runtime/runtime.cpp``, ``fbam_st_*``) implements
the same format in C++ for callers outside Python.
"""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, Iterable, Mapping

import numpy as np
import torch

_TO_ST = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16",
          torch.int32: "I32", torch.int64: "I64", torch.uint8: "U8", torch.bool: "BOOL"}
if hasattr(torch, "uint32"):
    _TO_ST[torch.uint32] = "U32"
    _TO_ST[torch.uint64] = "U64"
_FROM_ST = {v: k for k, v in _TO_ST.items()}
_ITEMSIZE = {"F32": 4, "F16": 2, "BF16": 2, "I32": 4, "I64": 8, "U32": 4, "U64": 8, "U8": 1, "BOOL": 1}


def _bytes_of(t: torch.Tensor) -> bytes:
    t = t.detach().contiguous().cpu()
    if t.numel() == 0:
        return b""
    return t.view(torch.uint8).numpy().tobytes() if t.dim() > 0 else t.reshape(1).view(torch.uint8).numpy().tobytes()


def save_file(tensors: Mapping[str, torch.Tensor], path: str, metadata: Mapping[str, str] | None = None) -> None:
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    names = sorted(tensors)
    for name in names:
        t = tensors[name]
        if t.dtype not in _TO_ST:
            raise TypeError(f"Unsupported dtype {t.dtype} for tensor '{name}'")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _TO_ST[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in names:
            f.write(_bytes_of(tensors[name]))
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


def read_header(path: str):
    with open(path, "rb") as f:
        raw = f.read(8)
        if len(raw) != 8:
            raise ValueError(f"{path}: truncated safetensors header")
        (n,) = struct.unpack("<Q", raw)
        if n > os.path.getsize(path) - 8:
            raise ValueError(f"{path}: header length {n} exceeds file size")
        header = json.loads(f.read(n).decode("utf-8"))
    return header, 8 + n


def load_file(path: str, pinned: bool = False) -> Dict[str, torch.Tensor]:
    header, base = read_header(path)
    out: Dict[str, torch.Tensor] = {}
    data = np.memmap(path, dtype=np.uint8, mode="r", offset=base) if os.path.getsize(path) > base else np.zeros(0, np.uint8)
    for name, info in header.items():
        if name == "__metadata__":
            continue
        st = info["dtype"]
        if st not in _FROM_ST:
            raise TypeError(f"{path}: tensor '{name}' has unsupported dtype {st}")
        lo, hi = info["data_offsets"]
        shape = tuple(info["shape"])
        count = int(np.prod(shape)) if shape else 1
        if hi - lo != count * _ITEMSIZE[st]:
            raise ValueError(f"{path}: tensor '{name}' byte range does not match its shape")
        buf = torch.empty(hi - lo, dtype=torch.uint8, pin_memory=pinned and torch.cuda.is_available())
        if hi > lo:
            buf.numpy()[:] = data[lo:hi]
        out[name] = buf.view(_FROM_ST[st]).reshape(shape)
    return out


def load_inplace(path: str, targets: Mapping[str, torch.Tensor], names: Iterable[str] | None = None) -> None:
    """Copies stored tensors into ``targets`` (dtype and shape must match exactly)."""
    loaded = load_file(path)
    for name in (names if names is not None else targets.keys()):
        if name not in loaded:
            raise KeyError(f"{path}: tensor '{name}' not found")
        src, dst = loaded[name], targets[name]
        if src.dtype != dst.dtype or tuple(src.shape) != tuple(dst.shape):
            raise ValueError(f"{path}: tensor '{name}' is {src.dtype}{tuple(src.shape)}, "
                             f"expected {dst.dtype}{tuple(dst.shape)}")
        dst.copy_(src)

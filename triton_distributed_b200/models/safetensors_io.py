"""A dependency-free reader / writer of the safetensors format, with shard-aware loading.

File format: 8-byte little-endian header length, a JSON header ``{name: {dtype, shape, data_offsets}}``, then the raw
little-endian tensor bytes.  ``ShardedCheckpoint`` understands ``model.safetensors.index.json`` (multi-file
checkpoints) and copies only the slice a rank needs (rows / columns of a 2-D weight) from the memory map, so a
TP rank never materialises a full weight.  Replaces the reference's use of ``AutoModelForCausalLM.from_pretrained``
(python/triton_dist/models/utils.py:108-170) for weight loading.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Optional, Tuple

import numpy as np
import torch

_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "I64": (torch.int64, 8), "I32": (torch.int32, 4), "I16": (torch.int16, 2), "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1), "F8_E4M3": (torch.float8_e4m3fn, 1), "F8_E5M2": (torch.float8_e5m2, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        (n,) = struct.unpack("<Q", self._f.read(8))
        self.header = json.loads(self._f.read(n).decode("utf-8"))
        self.metadata = self.header.pop("__metadata__", {})
        self.data_start = 8 + n
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)

    def keys(self) -> Iterable[str]:
        return self.header.keys()

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        e = self.header[name]
        return _DTYPES[e["dtype"]][0], tuple(e["shape"])

    def get(self, name: str, rows: Optional[Tuple[int, int]] = None, cols: Optional[Tuple[int, int]] = None) -> torch.Tensor:
        """Tensor ``name``; for 2-D tensors optionally only ``rows=(r0, r1)`` and/or ``cols=(c0, c1)``."""
        e = self.header[name]
        dtype, esz = _DTYPES[e["dtype"]]
        shape = tuple(e["shape"])
        b0, b1 = e["data_offsets"]
        buf = memoryview(self._mm)[self.data_start + b0:self.data_start + b1]
        flat = torch.frombuffer(buf, dtype=torch.uint8)
        if rows is not None and len(shape) >= 1:
            row_bytes = int(np.prod(shape[1:], dtype=np.int64)) * esz
            flat = flat[rows[0] * row_bytes:rows[1] * row_bytes]
            shape = (rows[1] - rows[0],) + shape[1:]
        t = flat.view(dtype).reshape(shape)
        if cols is not None:
            t = t[:, cols[0]:cols[1]]
        return t.clone()

    def close(self):
        self._mm.close()
        self._f.close()


def save_file(tensors: Dict[str, torch.Tensor], path: str, metadata: Optional[Dict[str, str]] = None):
    header, off, blobs = {}, 0, []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    if metadata:
        header["__metadata__"] = metadata
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


class ShardedCheckpoint:
    """All ``*.safetensors`` files of a directory behind one ``get``."""

    def __init__(self, directory: str):
        self.directory = directory
        self.files: Dict[str, SafetensorsFile] = {}
        self.where: Dict[str, str] = {}
        idx = os.path.join(directory, "model.safetensors.index.json")
        if os.path.exists(idx):
            with open(idx) as f:
                self.where = dict(json.load(f)["weight_map"])
        else:
            for fn in sorted(os.listdir(directory)):
                if fn.endswith(".safetensors"):
                    sf = self._file(fn)
                    for k in sf.keys():
                        self.where[k] = fn

    def _file(self, fn: str) -> SafetensorsFile:
        if fn not in self.files:
            self.files[fn] = SafetensorsFile(os.path.join(self.directory, fn))
        return self.files[fn]

    def __contains__(self, name: str) -> bool:
        return name in self.where

    def get(self, name: str, rows=None, cols=None) -> torch.Tensor:
        return self._file(self.where[name]).get(name, rows, cols)

    def shape(self, name: str) -> Tuple[int, ...]:
        return self._file(self.where[name]).info(name)[1]

    def get_row_shard(self, name: str, rank: int, world: int) -> torch.Tensor:
        n = self.shape(name)[0] // world
        return self.get(name, rows=(rank * n, (rank + 1) * n))

    def get_col_shard(self, name: str, rank: int, world: int) -> torch.Tensor:
        n = self.shape(name)[1] // world
        return self.get(name, cols=(rank * n, (rank + 1) * n))

    def close(self):
        for f in self.files.values():
            f.close()
        self.files.clear()

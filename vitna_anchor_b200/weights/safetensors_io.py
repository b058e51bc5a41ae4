"""Reading and writing the safetensors container.

The file is an 8-byte little-endian header length, a JSON directory
(name -> dtype, shape, data_offsets) and the tensors' bytes.  Every entry is
checked before anything is used, as the reference's reader does
(engine/src/safetensors.c:105-191): a known dtype, at most 8 dimensions, a
byte range inside the file that equals the number of elements times the
element size.  `__metadata__` is skipped.
"""
from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from typing import Dict, Mapping, Tuple

import numpy as np
import torch


class CheckpointError(ValueError):
    """The checkpoint file is malformed or does not fit the model."""


# dtype name -> (torch dtype, element size).  Integer tables come back as int32.
_DTYPES = {
    "F32": (torch.float32, 4),
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
}
_NAMES = {torch.float32: "F32", torch.bfloat16: "BF16", torch.float16: "F16", torch.int32: "I32"}


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    begin: int
    end: int


class SafetensorsFile:
    """A memory-mapped safetensors file; tensors are read by name."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise CheckpointError(f"cannot open {path}: {e.strerror}") from None
        self._f.seek(0, 2)
        size = self._f.tell()
        if size < 8:
            raise CheckpointError(f"{path}: too short to be a safetensors file")
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._map[:8])
        if hlen > size - 8:
            raise CheckpointError(f"{path}: the header is longer than the file")
        try:
            directory = json.loads(bytes(self._map[8:8 + hlen]).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise CheckpointError(f"{path}: the header is not JSON ({e})") from None
        if not isinstance(directory, dict):
            raise CheckpointError(f"{path}: the header is not an object")
        self._base = 8 + hlen
        data_len = size - self._base
        self.entries: Dict[str, TensorEntry] = {}
        for name, d in directory.items():
            if name == "__metadata__":
                continue
            try:
                dtype, shape, (lo, hi) = d["dtype"], tuple(int(s) for s in d["shape"]), d["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise CheckpointError(f"{path}: the entry of {name} is malformed") from None
            if dtype not in _DTYPES:
                raise CheckpointError(f"{path}: tensor {name} has dtype {dtype}, which is not supported")
            if len(shape) > 8 or any(s < 0 for s in shape):
                raise CheckpointError(f"{path}: tensor {name} has a bad shape")
            numel = int(np.prod(shape, dtype=np.int64)) if shape else 1
            if not (0 <= lo <= hi <= data_len) or hi - lo != numel * _DTYPES[dtype][1]:
                raise CheckpointError(f"{path}: the bytes of tensor {name} do not match its shape")
            self.entries[name] = TensorEntry(name, dtype, shape, lo, hi)

    def names(self):
        return list(self.entries)

    def read(self, name: str) -> torch.Tensor:
        """A host copy of the tensor, in its stored dtype (64-bit integers
        become int32; half floats stay as they are)."""
        e = self.entries[name]
        tdtype, _ = _DTYPES[e.dtype]
        buf = bytearray(self._map[self._base + e.begin:self._base + e.end])
        if not buf:
            t = torch.empty(e.shape, dtype=tdtype)
        else:
            t = torch.frombuffer(buf, dtype=tdtype).reshape(e.shape)
        if tdtype == torch.int64:
            t = t.to(torch.int32)
        return t

    def close(self):
        self._map.close()
        self._f.close()


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor]) -> None:
    """Write host tensors (float32, bfloat16, float16, int32) in the order given."""
    directory, blobs, off = {}, [], 0
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise CheckpointError(f"tensor {name}: dtype {t.dtype} cannot be written")
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        directory[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    header = json.dumps(directory, separators=(",", ":")).encode("utf-8")
    header += b" " * ((8 - len(header) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(header)))
        f.write(header)
        for raw in blobs:
            f.write(raw)

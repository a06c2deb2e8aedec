"""Reader and writer of the safetensors container, from its published layout:
an 8-byte little-endian header length, a JSON header
{name: {"dtype", "shape", "data_offsets": [begin, end]}}, then the raw bytes.
Tensors are read through a memory map, one at a time."""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path

import numpy as np
import torch

# container dtype -> (torch dtype, numpy dtype used to view the bytes)
DTYPES = {
    "F32": (torch.float32, np.float32),
    "BF16": (torch.bfloat16, np.uint16),
    "F16": (torch.float16, np.float16),
    "I32": (torch.int32, np.int32),
    "I64": (torch.int64, np.int64),
}
_NAMES = {v[0]: k for k, v in DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """Header of one file plus lazy access to its tensors."""

    def __init__(self, path):
        self.path = Path(path)
        with open(self.path, "rb") as f:
            head = f.read(8)
            if len(head) < 8:
                raise SafetensorsError(f"{self.path}: shorter than a safetensors header")
            (n,) = struct.unpack("<Q", head)
            size = self.path.stat().st_size
            if n <= 0 or 8 + n > size:
                raise SafetensorsError(f"{self.path}: header length {n} exceeds the file size {size}")
            try:
                header = json.loads(f.read(n))
            except json.JSONDecodeError as e:
                raise SafetensorsError(f"{self.path}: header is not JSON: {e}") from e
        if not isinstance(header, dict):
            raise SafetensorsError(f"{self.path}: header is not an object")
        self.metadata = header.pop("__metadata__", {})
        self.data_start = 8 + n
        self.entries = {}
        for name, meta in header.items():
            try:
                dtype, shape, (lo, hi) = meta["dtype"], tuple(int(s) for s in meta["shape"]), meta["data_offsets"]
            except (KeyError, TypeError, ValueError) as e:
                raise SafetensorsError(f"{self.path}: malformed entry for {name!r}") from e
            if self.data_start + hi > size or lo > hi:
                raise SafetensorsError(f"{self.path}: data of {name!r} lies outside the file")
            self.entries[name] = (dtype, shape, lo, hi)
        self._map = None

    def names(self):
        return list(self.entries)

    def info(self, name):
        dtype, shape, _, _ = self.entries[name]
        return dtype, shape

    def read(self, name) -> torch.Tensor:
        """CPU tensor that owns its memory, in the stored dtype."""
        dtype, shape, lo, hi = self.entries[name]
        if dtype not in DTYPES:
            raise SafetensorsError(f"{self.path}: unsupported dtype {dtype} of {name!r}")
        tdtype, ndtype = DTYPES[dtype]
        count = 1
        for s in shape:
            count *= s
        if (hi - lo) != count * np.dtype(ndtype).itemsize:
            raise SafetensorsError(f"{self.path}: {name!r} has {hi - lo} bytes for shape {shape} of {dtype}")
        if self._map is None:
            with open(self.path, "rb") as f:
                self._map = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        arr = np.frombuffer(self._map, dtype=ndtype, count=count, offset=self.data_start + lo).copy()
        t = torch.from_numpy(arr)
        if tdtype == torch.bfloat16:
            t = t.view(torch.bfloat16)
        return t.reshape(shape)

    def close(self):
        if self._map is not None:
            self._map.close()
            self._map = None


def write_safetensors(path, tensors: dict, metadata=None):
    """Write CPU tensors under their names, in the order given."""
    header, offset, blobs = {}, 0, []
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store {t.dtype} ({name})")
        raw = (t.view(torch.int16) if t.dtype == torch.bfloat16 else t).numpy().tobytes()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for raw in blobs:
            f.write(raw)

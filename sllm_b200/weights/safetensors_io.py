"""Own reader and writer of the safetensors container.

Layout (as the reference's dependency-free reader checks it,
loaders/safetensors_reader.py:82-139): 8 bytes little-endian header length, a
JSON object ``name -> {dtype, shape, data_offsets:[lo,hi)}`` (plus an optional
``__metadata__``), then the tensors' bytes.  Offsets are relative to the end of
the header; ``hi-lo`` must equal ``prod(shape)*itemsize`` and lie in the file.

Tensors come back as torch CPU tensors that alias a memory map of the file, in
the dtype they are stored in: bfloat16 stays bfloat16 (the reference widens
everything to float32, loaders/fp8.py:58-64, which doubles host memory), a
32-bit tensor stays 32-bit, integer tables come back as int32.
"""

from __future__ import annotations

import json
import mmap
import os
import struct

import torch

MAX_HEADER_BYTES = 256 * 1024 * 1024      # loaders/safetensors_reader.py:51

_DTYPES = {
    "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2), "F32": (torch.float32, 4),
    "F64": (torch.float64, 8), "I32": (torch.int32, 4), "I64": (torch.int64, 8),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    """The file is not a well-formed safetensors container."""


def parse_header(path: str):
    """(entries, data_start, file_size); entries: name -> (dtype_name, shape, lo, hi)."""
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) != 8:
            raise SafetensorsError(f"{path}: shorter than the 8-byte header length")
        (n,) = struct.unpack("<Q", head)
        if n > MAX_HEADER_BYTES or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} is not plausible for a file of {size} bytes")
        try:
            header = json.loads(f.read(n))
        except (json.JSONDecodeError, UnicodeDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not JSON ({e})") from None
    if not isinstance(header, dict):
        raise SafetensorsError(f"{path}: header is not a JSON object")
    start = 8 + n
    entries = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        try:
            dtype, shape, (lo, hi) = meta["dtype"], tuple(int(s) for s in meta["shape"]), meta["data_offsets"]
        except (KeyError, TypeError, ValueError):
            raise SafetensorsError(f"{path}: entry {name!r} lacks dtype/shape/data_offsets") from None
        if dtype not in _DTYPES:
            raise SafetensorsError(f"{path}: entry {name!r} has unsupported dtype {dtype!r}")
        count = 1
        for s in shape:
            count *= s
        if hi - lo != count * _DTYPES[dtype][1]:
            raise SafetensorsError(f"{path}: entry {name!r}: {hi - lo} bytes stored, shape {shape} "
                                   f"of {dtype} needs {count * _DTYPES[dtype][1]}")
        if lo < 0 or start + hi > size:
            raise SafetensorsError(f"{path}: entry {name!r} reaches past the end of the file (truncated?)")
        entries[name] = (dtype, shape, lo, hi)
    return entries, start, size


class SafetensorsFile:
    """One file, memory-mapped; tensors are views, read when touched."""

    def __init__(self, path: str):
        self.path = path
        self.entries, self._start, size = parse_header(path)
        self._f = open(path, "rb")
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_COPY) if size else None

    def names(self):
        return list(self.entries)

    def shape_of(self, name: str):
        return self.entries[name][1]

    def dtype_of(self, name: str) -> str:
        return self.entries[name][0]

    def tensor(self, name: str) -> torch.Tensor:
        dtype, shape, lo, hi = self.entries[name]
        tdtype, item = _DTYPES[dtype]
        count = (hi - lo) // item
        if count == 0:
            return torch.empty(shape, dtype=tdtype)
        t = torch.frombuffer(self._map, dtype=tdtype, count=count, offset=self._start + lo)
        t = t.reshape(shape)
        if tdtype in (torch.int64, torch.int16, torch.int8, torch.uint8):
            t = t.to(torch.int32)
        return t

    def close(self):
        # tensors handed out alias the map; it is closed when they are gone
        self._f.close()


def write_safetensors(path: str, tensors: dict, metadata: dict | None = None) -> None:
    """Write CPU tensors under their names, in the order given, 8-byte aligned header."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store {name!r} of dtype {t.dtype}")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + n]}
        offset += n
        blobs.append(t)
    raw = json.dumps(header, separators=(",", ":")).encode()
    raw += b" " * (-len(raw) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for t in blobs:
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else t.reshape(1).view(torch.uint8).numpy().tobytes())

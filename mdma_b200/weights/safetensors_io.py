"""A small reader and writer for the safetensors container.

File = 8-byte little-endian header length, a JSON header
{name: {dtype, shape, data_offsets:[begin,end]}} and the tensor bytes.  The
reader checks what the reference's header pass checks before any tensor is
touched (src/model/weights.rs:26-70): the header is at most 100 MB and lies
inside the file, every tensor's byte range matches its shape and dtype, and
the tensors fill the file exactly.  Tensors are returned as views of one
memory map, so nothing is copied until a tensor is uploaded.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Iterable

import torch

MAX_HEADER_BYTES = 100_000_000

_DTYPES = {
    "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class CheckpointError(ValueError):
    """The file is not a well-formed safetensors container."""


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: tuple
    begin: int      # byte offsets inside the data section
    end: int
    file: str


def _numel(shape: Iterable[int]) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


def read_header(path: str) -> tuple[dict[str, TensorEntry], int]:
    """Parse and validate the header; returns (entries, offset of the data section)."""
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        prefix = f.read(8)
        if len(prefix) != 8:
            raise CheckpointError(f"{path}: shorter than a safetensors prefix")
        (n,) = struct.unpack("<Q", prefix)
        if n > MAX_HEADER_BYTES or n > size - 8:
            raise CheckpointError(f"{path}: header claims {n} bytes")
        raw = f.read(n)
    try:
        header = json.loads(raw)
    except (json.JSONDecodeError, UnicodeDecodeError) as e:
        raise CheckpointError(f"{path}: header is not JSON: {e}") from None
    if not isinstance(header, dict):
        raise CheckpointError(f"{path}: header must be a JSON object")
    data_len = size - 8 - n
    entries: dict[str, TensorEntry] = {}
    spans = []
    for name, info in header.items():
        if name == "__metadata__":
            continue
        try:
            dtype_name, shape, (begin, end) = info["dtype"], tuple(info["shape"]), info["data_offsets"]
        except (KeyError, TypeError, ValueError):
            raise CheckpointError(f"{path}: malformed entry for tensor {name!r}") from None
        if dtype_name not in _DTYPES:
            raise CheckpointError(f"{path}: tensor {name!r} has unsupported dtype {dtype_name!r}")
        dtype, width = _DTYPES[dtype_name]
        if any((not isinstance(s, int)) or s < 0 for s in shape):
            raise CheckpointError(f"{path}: tensor {name!r} has a bad shape {shape}")
        if not (0 <= begin <= end <= data_len) or end - begin != _numel(shape) * width:
            raise CheckpointError(
                f"{path}: tensor {name!r} spans bytes [{begin},{end}) but shape {shape} of "
                f"{dtype_name} needs {_numel(shape) * width} inside {data_len}")
        entries[name] = TensorEntry(name, dtype, shape, begin, end, path)
        spans.append((begin, end))
    spans.sort()
    cursor = 0
    for begin, end in spans:
        if begin != cursor:
            raise CheckpointError(f"{path}: tensors do not fill the file (gap or overlap at byte {cursor})")
        cursor = end
    if cursor != data_len:
        raise CheckpointError(f"{path}: tensors do not fill the file ({data_len - cursor} bytes left over)")
    return entries, 8 + n


class SafetensorsFile:
    """One opened file: validated entries plus a lazily created memory map."""

    def __init__(self, path: str):
        self.path = path
        self.entries, self._data_start = read_header(path)
        self._map = None

    def tensor(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        if self._map is None:
            with open(self.path, "rb") as f:
                self._map = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_COPY)
        if e.end == e.begin:
            return torch.empty(e.shape, dtype=e.dtype)
        buf = memoryview(self._map)[self._data_start + e.begin:self._data_start + e.end]
        return torch.frombuffer(buf, dtype=e.dtype).reshape(e.shape)


def write_safetensors(path: str, tensors: dict[str, torch.Tensor], metadata: dict | None = None) -> None:
    """Write `tensors` (CPU, any supported dtype) in name order."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise CheckpointError(f"cannot store tensor {name!r} of dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * ((8 - len(raw) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else
                        t.reshape(1).view(torch.uint8).numpy().tobytes())

"""Reader and writer of the safetensors container, by hand: 8 bytes of little-endian
header length, a JSON header {name: {dtype, shape, data_offsets}}, then the bytes.

It stands where the reference parses GGUF by hand and maps the file
(src/gguf/reader.rs:32-58, src/tensor/storage.rs:15-20): tensors are views of one
memory map and are found by name.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from typing import Dict, Iterable, List, Tuple

import torch

_DTYPES = {
    "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class WeightFileError(ValueError):
    """A file that is not a readable safetensors container."""


class SafetensorsFile:
    """One mapped file.  `entries[name] = (dtype string, shape, begin, end)`."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise WeightFileError(f"{path}: {size} bytes is too short for a safetensors header")
        self._f = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise WeightFileError(f"{path}: header length {hlen} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise WeightFileError(f"{path}: header is not JSON ({e})") from None
        self.metadata = header.pop("__metadata__", {})
        self._base = 8 + hlen
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self.entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, e in header.items():
            dt, shape = e.get("dtype"), tuple(int(s) for s in e.get("shape", []))
            b, en = (int(x) for x in e.get("data_offsets", (0, -1)))
            if dt not in _DTYPES:
                raise WeightFileError(f"{path}: tensor '{name}' has unsupported dtype {dt!r}")
            n = 1
            for s in shape:
                n *= s
            if b < 0 or en < b or self._base + en > size or en - b != n * _DTYPES[dt][1]:
                raise WeightFileError(f"{path}: tensor '{name}' offsets [{b},{en}) do not match shape "
                                      f"{list(shape)} {dt} or leave the file ({size - self._base} data bytes)")
            self.entries[name] = (dt, shape, b, en)

    def names(self) -> List[str]:
        return list(self.entries)

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.entries[name][0]][0]

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.entries[name][1]

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that views the map (copy it before the file is closed)."""
        dt, shape, b, e = self.entries[name]
        if e == b:
            return torch.empty(shape, dtype=_DTYPES[dt][0])
        buf = memoryview(self._map)[self._base + b:self._base + e]
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)       # the map is read-only; nobody writes to it
            return torch.frombuffer(buf, dtype=_DTYPES[dt][0]).reshape(shape)


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]], metadata=None) -> None:
    """Writes tensors in the order given; each tensor's bytes start on an 8-byte boundary
    of the data section (the header is padded with spaces)."""
    items = [(n, t.detach().cpu().contiguous()) for n, t in tensors]
    header, off = {}, 0
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for n, t in items:
        if t.dtype not in _NAMES:
            raise WeightFileError(f"cannot store dtype {t.dtype} of '{n}'")
        nbytes = t.numel() * t.element_size()
        header[n] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for _, t in items:
            if t.numel():
                f.write(memoryview(t.reshape(-1).view(torch.uint8).numpy()))


def open_model_files(folder: str) -> List[SafetensorsFile]:
    """model.safetensors, or the shards that model.safetensors.index.json lists."""
    single = os.path.join(folder, "model.safetensors")
    index = os.path.join(folder, "model.safetensors.index.json")
    if os.path.exists(single):
        return [SafetensorsFile(single)]
    if os.path.exists(index):
        with open(index) as f:
            shards = sorted(set(json.load(f)["weight_map"].values()))
        return [SafetensorsFile(os.path.join(folder, s)) for s in shards]
    raise WeightFileError(f"{folder}: neither model.safetensors nor model.safetensors.index.json")

"""Reader and writer of the safetensors container: 8 bytes of little-endian header
length, a JSON header {name: {dtype, shape, data_offsets}}, then the bytes.

The reader is native (csrc/safetensors_file.cu): it parses the header, maps the file,
checks every entry and moves tensors to the device through pinned staging buffers,
converting on the device.  It stands where the reference parses GGUF by hand and maps
the file (src/gguf/reader.rs:32-58, src/tensor/storage.rs:15-20): tensors are views
of one memory map and are found by name.  The writer (for the random-weights mode;
the reference has none) is a few lines of Python.
"""
from __future__ import annotations

import ctypes
import json
import os
import struct
import warnings
from typing import Dict, Iterable, List, Tuple

import torch

from .. import native

_DTYPES = {
    "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}
_KEEP = {torch.float32: 0, torch.bfloat16: 1, torch.int32: 2}

_C, _V, _LP = ctypes.c_char_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_longlong)
native.register_signature("gb_st_open", [_C, ctypes.POINTER(_V)])
native.register_signature("gb_st_close", [_V])
native.register_signature("gb_st_count", [_V])
native.register_signature("gb_st_entry", [_V, ctypes.c_int, ctypes.POINTER(_C), ctypes.POINTER(_C), ctypes.POINTER(ctypes.c_int),
                                          ctypes.POINTER(_LP), ctypes.POINTER(_V), _LP])
native.register_signature("gb_st_metadata_count", [_V])
native.register_signature("gb_st_metadata", [_V, ctypes.c_int, ctypes.POINTER(_C), ctypes.POINTER(_C)])
native.register_signature("gb_st_upload", [_V, ctypes.c_int, _V, ctypes.c_int, _V])


class WeightFileError(ValueError):
    """A file that is not a readable safetensors container."""


class SafetensorsFile:
    """One mapped file.  `entries[name] = (dtype string, shape, index in the file's table)`."""

    def __init__(self, path: str):
        self.path = path
        self._lib = native.library()
        handle = _V()
        if self._lib.gb_st_open(os.fsencode(path), ctypes.byref(handle)):
            raise WeightFileError(self._lib.gb_last_error().decode("utf-8", "replace"))
        self._h = handle
        self.entries: Dict[str, Tuple[str, Tuple[int, ...], int]] = {}
        self._bytes: Dict[str, Tuple[int, int]] = {}
        name, dtype, ndim, shape, addr, nbytes = _C(), _C(), ctypes.c_int(), _LP(), _V(), ctypes.c_longlong()
        for i in range(self._lib.gb_st_count(self._h)):
            self._lib.gb_st_entry(self._h, i, ctypes.byref(name), ctypes.byref(dtype), ctypes.byref(ndim), ctypes.byref(shape),
                                  ctypes.byref(addr), ctypes.byref(nbytes))
            n = name.value.decode("utf-8")
            self.entries[n] = (dtype.value.decode("ascii"), tuple(int(shape[d]) for d in range(ndim.value)), i)
            self._bytes[n] = (addr.value or 0, int(nbytes.value))
        self.metadata: Dict[str, str] = {}
        key, value = _C(), _C()
        for i in range(self._lib.gb_st_metadata_count(self._h)):
            self._lib.gb_st_metadata(self._h, i, ctypes.byref(key), ctypes.byref(value))
            self.metadata[key.value.decode("utf-8")] = value.value.decode("utf-8")

    def __del__(self):                                          # unmaps once no tensor views the file any more
        h, self._h = getattr(self, "_h", None), None
        if h is not None:
            self._lib.gb_st_close(h)

    def names(self) -> List[str]:
        return list(self.entries)

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.entries[name][0]][0]

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.entries[name][1]

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that views the map (copy it before the file is closed)."""
        dt, shape, _ = self.entries[name]
        addr, nbytes = self._bytes[name]
        if nbytes == 0:
            return torch.empty(shape, dtype=_DTYPES[dt][0])
        buf = (ctypes.c_uint8 * nbytes).from_address(addr)
        buf._file = self                                        # the map lives as long as any tensor views it
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)       # the map is read-only; nobody writes to it
            return torch.frombuffer(buf, dtype=_DTYPES[dt][0]).reshape(shape)

    def to_device(self, name: str, dtype: torch.dtype, device) -> torch.Tensor:
        """The tensor on a CUDA device, kept as float32, bfloat16 or int32: staged through pinned memory
        and converted on the device, in the current stream."""
        _, shape, index = self.entries[name]
        out = torch.empty(shape, dtype=dtype, device=device)
        with torch.cuda.device(out.device):
            if self._lib.gb_st_upload(self._h, index, out.data_ptr(), _KEEP[dtype], native.stream_ptr()):
                raise WeightFileError(self._lib.gb_last_error().decode("utf-8", "replace"))
        return out


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

"""Weights by tensor name, with one error that lists everything that is wrong.

Parts declare the tensors they need (`TensorRequest`: name in the file, shape,
optional or not, and for an optional tensor the name that stands in for it).  The
store checks all declarations against the source at once and raises one
`WeightError` naming missing tensors, tensors nobody asked for, and wrong shapes;
the reference stops at the first missing name and checks no shape
(src/model/llama.rs:98-117).

Storage dtypes: with `bfloat16`, 16-bit floats are kept as bfloat16 and a tensor
stored in 32-bit stays 32-bit; with `float32`, every float becomes 32-bit.  Integer
tables become int32.
"""
from __future__ import annotations

import fnmatch
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from .safetensors_io import SafetensorsFile, open_model_files


class WeightError(ValueError):
    def __init__(self, missing, unexpected, wrong_shape, where=""):
        self.missing, self.unexpected, self.wrong_shape = list(missing), list(unexpected), list(wrong_shape)
        lines = [f"weights of {where or 'the model'} do not match its configuration:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(
                f"{n}: expected {list(e)}, found {list(f)}" for n, e, f in self.wrong_shape))
        super().__init__("\n".join(lines))


@dataclass(frozen=True)
class TensorRequest:
    name: str
    shape: Tuple[int, ...]
    optional: bool = False
    fallback: Optional[str] = None      # another tensor's name that is used when this one is absent
    # what the random-weights mode writes for it: "normal" (N(0, 0.02)), "ones", "zeros", or None (nothing:
    # the tensor is left out of the folder and its fallback stands in)
    init: Optional[str] = "normal"


class TensorSource:
    """Names, shapes and tensors of a model folder or of a dict in memory."""

    def __init__(self, tensors: Optional[Dict[str, torch.Tensor]] = None, files: Optional[List[SafetensorsFile]] = None,
                 where: str = ""):
        self.where = where
        self._tensors = tensors or {}
        self._files = files or []
        self._index: Dict[str, SafetensorsFile] = {}
        dup = []
        for f in self._files:
            for n in f.names():
                if n in self._index:
                    dup.append(n)
                self._index[n] = f
        if dup:
            raise WeightError([], [f"{n} (stored in more than one shard)" for n in dup], [], where)

    @classmethod
    def from_folder(cls, folder: str) -> "TensorSource":
        return cls(files=open_model_files(folder), where=folder)

    def names(self) -> List[str]:
        return list(self._tensors) + list(self._index)

    def has(self, name: str) -> bool:
        return name in self._tensors or name in self._index

    def shape(self, name: str) -> Tuple[int, ...]:
        if name in self._tensors:
            return tuple(self._tensors[name].shape)
        return self._index[name].shape(name)

    def get(self, name: str) -> torch.Tensor:
        if name in self._tensors:
            return self._tensors[name]
        return self._index[name].tensor(name)

    def dtype(self, name: str) -> torch.dtype:
        if name in self._tensors:
            return self._tensors[name].dtype
        return self._index[name].dtype(name)

    def to_device(self, name: str, dtype: torch.dtype, device) -> torch.Tensor:
        """The tensor on `device` as `dtype`; tensors of a file on their way to a CUDA device are staged and
        converted by the native reader."""
        if name not in self._tensors and torch.device(device).type == "cuda":
            return self._index[name].to_device(name, dtype, device)
        return self.get(name).to(device=device, dtype=dtype).contiguous()


def storage_dtype(stored: torch.dtype, mode: torch.dtype) -> torch.dtype:
    """The dtype a tensor is kept in on the device (see the module text)."""
    if stored.is_floating_point:
        if mode == torch.float32:
            return torch.float32
        return torch.float32 if stored in (torch.float32, torch.float64) else torch.bfloat16
    return torch.int32


class WeightStore:
    """Checks requests against a source, then hands out device tensors."""

    def __init__(self, source: TensorSource, mode: torch.dtype, device):
        self.source, self.mode, self.device = source, mode, device
        self._cache: Dict[str, torch.Tensor] = {}

    def check(self, requests: Iterable[TensorRequest], allow_unused: Iterable[str] = ()) -> None:
        """allow_unused: names or shell-style patterns of tensors a folder may hold although nobody asks
        for them (buffers that older exports keep beside the parameters)."""
        missing, wrong, asked = [], [], set()
        patterns = list(allow_unused)
        for r in requests:
            name = r.name
            if not self.source.has(name):
                if r.fallback is not None and self.source.has(r.fallback):
                    name = r.fallback
                elif r.optional and r.fallback is None:
                    continue
                else:
                    missing.append(r.name)
                    continue
            asked.add(name)
            found = self.source.shape(name)
            if tuple(found) != tuple(r.shape):
                wrong.append((name, tuple(r.shape), tuple(found)))
        unexpected = sorted(n for n in self.source.names()
                            if n not in asked and not any(fnmatch.fnmatchcase(n, pat) for pat in patterns))
        if missing or unexpected or wrong:
            raise WeightError(sorted(set(missing)), unexpected, wrong, self.source.where)

    def resolve(self, r: TensorRequest) -> Optional[str]:
        if self.source.has(r.name):
            return r.name
        if r.fallback is not None and self.source.has(r.fallback):
            return r.fallback
        return None

    def get(self, r: TensorRequest) -> Optional[torch.Tensor]:
        """The tensor on the device in its storage dtype, or None for an absent optional
        one.  Asking twice for one name (a tied head) gives the same tensor."""
        name = self.resolve(r)
        if name is None:
            return None
        if name not in self._cache:
            keep = storage_dtype(self.source.dtype(name), self.mode)
            self._cache[name] = self.source.to_device(name, keep, self.device)
        return self._cache[name]

    def release(self) -> None:
        """Forget the handed-out tensors (parts keep what they need)."""
        self._cache.clear()

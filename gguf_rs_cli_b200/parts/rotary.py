"""Rotary position encoding as a table of inverse frequencies plus a width and a
pairing; the rotation itself happens in the kernel that also writes the cache.

f_i = theta^(-2i/rotary_dim), angle = position * f_i, pairs (i, i + rotary_dim/2)
("half", src/math/rope.rs:6-13) or (2i, 2i+1) ("interleaved").  Frequency scaling is
not in the reference (src/model/config.rs:43 reads the base only); "llama3" rescales
by wavelength l = 2*pi/f against the original context length `orig`:
l < orig/high_freq_factor keeps f; l > orig/low_freq_factor gives f/factor; between
them s = (orig/l - low)/(high - low), f <- (1-s) f/factor + s f.  "linear" divides
every f by factor.  The table is built in 64-bit and kept in 32-bit.
"""
from __future__ import annotations

import math
from typing import List

import torch

from .base import Part
from .registry import register_position


def inverse_frequencies(rotary_dim: int, theta: float, scaling=None) -> List[float]:
    f = [float(theta) ** (-2.0 * i / rotary_dim) for i in range(rotary_dim // 2)]
    if not scaling:
        return f
    kind = scaling.get("rope_type", scaling.get("type"))
    if kind in (None, "default"):
        return f
    factor = float(scaling["factor"])
    if kind == "linear":
        return [x / factor for x in f]
    if kind == "llama3":
        low, high = float(scaling.get("low_freq_factor", 1.0)), float(scaling.get("high_freq_factor", 4.0))
        orig = float(scaling.get("original_max_position_embeddings", 8192))
        out = []
        for x in f:
            wavelength = 2.0 * math.pi / x
            if wavelength < orig / high:
                out.append(x)
            elif wavelength > orig / low:
                out.append(x / factor)
            else:
                s = (orig / wavelength - low) / (high - low)
                out.append((1.0 - s) * x / factor + s * x)
        return out
    raise ValueError(f"rope scaling of type {kind!r} is not known (llama3, linear, default)")


@register_position("rope")
class Rotary(Part):
    """params: head_dim, rotary_dim, theta, pairing ("half" or "interleaved"), scaling."""

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.rotary_dim = int(self.p.get("rotary_dim", self.p["head_dim"]))
        if self.rotary_dim % 2 or self.rotary_dim > self.p["head_dim"]:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.p['head_dim']}")
        self.pairing = {"half": 0, "interleaved": 1}[self.p.get("pairing", "half")]
        table = inverse_frequencies(self.rotary_dim, self.p["theta"], self.p.get("scaling"))
        self.inv_freq = torch.tensor(table, dtype=torch.float64).to(torch.float32).to(device)

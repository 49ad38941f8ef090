"""Device sampling for the sequences of a step; see csrc/sampling.cu for the rules."""
from __future__ import annotations

from typing import Sequence

import torch

from .. import kernels
from .params import SamplingParams


class Sampler:
    """Draws one token per row of logits.  The sequences' recent-token rings and draw
    counters live in the cache's per-sequence state (`sampler.recent`, `sampler.count`)
    and are zeroed when a slot is opened."""

    def __init__(self, cache, device):
        self.recent = cache.states["sampler.recent"]
        self.count = cache.states["sampler.count"]
        self.device = device

    def sample(self, logits: torch.Tensor, slots: torch.Tensor, keys: torch.Tensor, params: SamplingParams,
               out: torch.Tensor) -> torch.Tensor:
        """logits float32 [n, V]; slots int32 [n]; keys int64 [n] (stream_key of each request);
        out int32 [>= n].  Launches on the current stream and does not synchronise."""
        return kernels.sample(logits, slots, keys, params.temperature, params.top_k, params.top_p, params.rep_penalty,
                              self.recent, self.count, out)

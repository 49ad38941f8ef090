"""Sampling options, with the reference's names and meanings (src/main.rs:24-31,48-49;
src/sampler.rs:35-79).  The defaults are the neutral ones (greedy, nothing cut, no
penalty); the command line sets the reference's own defaults."""
from __future__ import annotations

from dataclasses import dataclass

MASK64 = (1 << 64) - 1
_GOLDEN = 0x9E3779B97F4A7C15


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0      # <= 0: the largest logit
    top_k: int = 0                # 0: off
    top_p: float = 1.0            # 1: off
    rep_penalty: float = 1.0      # 1: off; applies to the last 64 emitted tokens
    seed: int = 42

    def validate(self) -> None:
        if self.top_k < 0:
            raise ValueError(f"top_k must be 0 (off) or positive, got {self.top_k}")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if not self.rep_penalty > 0.0:
            raise ValueError(f"rep_penalty must be positive, got {self.rep_penalty}")


def _splitmix64(z: int) -> int:
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
    return z ^ (z >> 31)


def stream_key(seed: int, request_index: int) -> int:
    """Key of one request's random stream, so that a request's draws do not depend on what
    else is in its batch.  As a signed 64-bit value for an int64 tensor."""
    k = _splitmix64((int(seed) + (int(request_index) + 1) * _GOLDEN) & MASK64)
    return k - (1 << 64) if k >= (1 << 63) else k

"""Interfaces of the parts and the objects a step hands them.

Every part is built from its `PartSpec` alone (sizes and constants in `spec.params`,
tensor names in `spec.tensors`), says which tensors it needs (`tensor_requests`),
takes them from the store (`load`), and computes on the tokens of one step.  No part
knows which model it is in.

Roles:
  norm          apply(stream, ctx, rows=None, absorbed=False) -> normalised rows in ctx.dtype; folds
                the stream's pending term into x (32-bit sum) on the way.  Optional `fold_weight()`
                gives its weight to a consumer that can multiply it into its own matrix
                (`absorb_input_norm(w) -> bool`); the block then calls apply(absorbed=True), which
                leaves the weight out and may return a DeferredNorm instead of rows
  position      gives the mixer what it needs to encode positions (for "rope": inv_freq,
                rotary_dim, pairing)
  mixer         kv_spec() -> KVSpec or None; state_spec() -> {name: (shape, dtype name)};
                forward(h, ctx, run) -> term [T, E] (or [S, T, E] partial sums) to add to x.
                A part with `accepts_residual = True` is called with residual=stream and may add
                its term to the stream itself (returning None)
  feed-forward  forward(h, ctx) -> term to add to x
  block         forward(stream, ctx, run): wires norms, mixer and feed-forward around x
  embedding     forward(tokens, ctx) -> float32 x [T, E]
  head          forward(h, ctx) -> float32 logits [rows, V]

Optional hooks of any part (a part without them works):
  plan(batch: HostBatch) -> {name: list of int}   index arrays the part lays out on the host for this
                step; they travel in the step's one host-to-device copy and come back as int32
                device tensors in ctx.plan_of(part)
  plan_key() -> hashable   parts with equal keys share one plan and one graph class (layers with the
                same constants); default: every part for itself
  graph_class   whether and how decode steps that contain the part may be captured in a CUDA graph:
                a hashable constant, or graph_class(batch) -> hashable, equal for steps whose launches
                (grids, buffer shapes, host-side branches, plan sizes) are the same; None or no
                attribute at all: never captured (a part that computes with host values each step)
  ctx.mark(label)          a time stamp after a stage, recorded when a step is profiled
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import torch

from ..cache.cache import Cache, KVSpec
from ..config.specs import PartSpec
from ..weights.loader import TensorRequest, WeightStore


class Part:
    def __init__(self, spec: PartSpec, dtype: torch.dtype, device):
        self.spec, self.dtype, self.device = spec, dtype, device
        self.p = spec.params

    def tensor_requests(self) -> List[TensorRequest]:
        return []

    def load(self, store: WeightStore) -> None:
        pass


class Workspace:
    """Buffers that live as long as the engine and are handed out by name, so that a
    step allocates nothing once its shapes have been seen (and a captured graph keeps
    valid addresses)."""

    def __init__(self, device):
        self.device = device
        self._bufs: Dict[Tuple, torch.Tensor] = {}

    def get(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        key = (name, tuple(int(s) for s in shape), dtype)
        t = self._bufs.get(key)
        if t is None:
            t = torch.empty(key[1], dtype=dtype, device=self.device)
            self._bufs[key] = t
        return t

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._bufs.values())


@dataclass
class HostBatch:
    """One step as the host sees it, for parts that plan there: the sequences' cache slots, their
    lengths before the step and the tokens each brings."""
    slots: Sequence[int]
    starts: Sequence[int]
    qlens: Sequence[int]
    decode: bool                  # every sequence brings exactly one token
    max_qlen: int
    max_kv: int                   # longest cached length after this step


def plan_key_of(part) -> Hashable:
    key = getattr(part, "plan_key", None)
    return key() if key else id(part)


@dataclass
class RunView:
    """What one entry of the run order sees of the cache: its group's geometry and its
    own K and V storage [pages, kv heads, PAGE, head_dim] (None when the mixer keeps no
    keys), plus the page tables of this step's sequences for that group."""
    index: int
    layer: int
    owns_cache: bool
    group: Optional[int] = None
    k: Optional[torch.Tensor] = None
    v: Optional[torch.Tensor] = None
    ring_pages: int = 1
    kv_spec: Optional[KVSpec] = None


@dataclass
class StepContext:
    """One step's batch on the device.  T tokens of B sequences, packed sequence after
    sequence; padding tokens have seq_of = -1 and padding sequences slot = -1."""
    T: int
    B: int
    dtype: torch.dtype
    tokens: torch.Tensor          # int32 [T]
    seq_of: torch.Tensor          # int32 [T]  row of the token's sequence in this step's tables
    pos: torch.Tensor             # int32 [T]  position of the token in its sequence
    slots: torch.Tensor           # int32 [B]  cache slot of each sequence (-1: padding)
    starts: torch.Tensor          # int32 [B]  cached length before this step
    qlens: torch.Tensor           # int32 [B]
    cu: torch.Tensor              # int32 [B+1] first token of each sequence in the packing
    tables: List[torch.Tensor]    # per cache group: int32 [B, table width]
    cache: Cache
    ws: Workspace
    decode: bool                  # every sequence brings exactly one token
    max_qlen: int
    max_kv: int                   # longest cached length after this step
    host: Dict = field(default_factory=dict)    # host copies for parts that plan on the host
    plans: Dict = field(default_factory=dict)   # plan key -> {name: int32 device tensor} (see plan_of)
    marks: Optional[List] = None                # (label, CUDA event) after each stage, when the step is profiled
    mark_detail: bool = True

    def state(self, name: str) -> torch.Tensor:
        """Fixed-size per-sequence state [slots, ...]; index it with ctx.slots."""
        return self.cache.states[name]

    def plan_of(self, part) -> Dict[str, torch.Tensor]:
        """The index arrays that `part.plan(batch)` laid out for this step, on the device."""
        return self.plans.get(plan_key_of(part), {})

    def mark(self, label: str) -> None:
        """A time stamp on the current stream after the stage `label`; nothing unless the step is profiled
        (the reference stamps its command buffer the same way, src/gpu/mod.rs:333-343)."""
        if self.marks is not None and self.mark_detail:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.marks.append((label, ev))


# Steps of at most this many tokens fold residual adds and norms into the products' epilogues (there the
# step is bound by launches and bandwidth); larger steps keep the separate norm kernel, whose cost the
# compute-bound products would otherwise carry in their epilogues.
FUSE_MAX_TOKENS = 128


class Stream:
    """The residual stream: x in float32 plus a term that has not been added yet.  The
    next norm adds it in 32-bit in the same kernel that normalises.

    A producer that adds its term to x itself (a product's residual epilogue, the embedding)
    may leave a shadow for the norm that follows: xb = bfloat16(x) and ssq [parts, T], partial
    sums of x^2 per token.  The shadow is valid while nothing is pending and x is unchanged."""

    def __init__(self, x: torch.Tensor):
        self.x = x
        self.pending: Optional[torch.Tensor] = None
        self.xb: Optional[torch.Tensor] = None
        self.ssq: Optional[torch.Tensor] = None
        self.ssq_parts = 0

    def drop_shadow(self) -> None:
        self.xb, self.ssq, self.ssq_parts = None, None, 0


@dataclass
class DeferredNorm:
    """Rows whose RMS norm has not been applied: the consumer (a product that has folded the
    norm's weight into its matrix) scales its results per token by
    1 / sqrt(sum_i ssq[i, t] / size + eps) instead."""
    xb: torch.Tensor
    ssq: torch.Tensor
    parts: int
    size: int
    eps: float

    @property
    def shape(self):
        return self.xb.shape

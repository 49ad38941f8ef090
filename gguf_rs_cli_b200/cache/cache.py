"""The cache: a slot for each live sequence, keys and values for every run of a layer
that needs them, each sequence with its own length, and beside it per-sequence
state of fixed size.

Runs with the same needs (KV heads, head size, all keys or a window of them) form
a group with storage of its own: K and V of shape
[runs of the group, pages, kv heads, PAGE positions, head_dim], so that one page of
one KV head is a contiguous [PAGE, head_dim] tile.  A sequence's positions map to
pages through its page table; a windowed group keeps only a ring of pages per
sequence (position p lives in table entry (p // PAGE) % ring_pages), sized so that
every key a step can still need is resident: window + the longest step - 1
positions.  What a slot holds is valid up to its length; pages and state are given
back when the sequence is closed and are used again without being cleared, except
the fixed-size state, which is zeroed when a slot is opened.

The reference keeps one sequence in per-layer buffers of the whole context and its
position in the caller (src/model/llama.rs:64-73, 179-186; src/main.rs:109).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

from .pool import PAGE, CacheError, CacheFull, FreeList, pages_for


@dataclass(frozen=True)
class KVSpec:
    """What one run of a mixer needs to keep per position."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None        # None: all keys; W: the last W positions


@dataclass
class CacheLayout:
    """kv[run index] for runs that own keys and values; states[name] = (shape, dtype
    name) of fixed-size per-sequence state."""
    kv: Dict[int, KVSpec] = field(default_factory=dict)
    states: Dict[str, Tuple[Tuple[int, ...], str]] = field(default_factory=dict)


class KVGroup:
    def __init__(self, index: int, spec: KVSpec, runs: List[int], n_pages: int, ring_pages: int, table_width: int):
        self.index, self.spec, self.runs = index, spec, runs
        self.n_pages, self.ring_pages, self.table_width = n_pages, ring_pages, table_width
        self.pool = FreeList(n_pages, f"page of group {index}")
        self.tables: Dict[int, List[int]] = {}
        self.k = None
        self.v = None

    def pages_needed(self, length: int) -> int:
        return min(pages_for(length), self.ring_pages)


class Cache:
    def __init__(self, layout: CacheLayout, n_slots: int, n_tokens: int, max_len: Optional[int] = None,
                 max_step_tokens: Optional[int] = None, dtype=None, device=None):
        """n_tokens: the most positions that live sequences hold together, each
        sequence rounded up to whole pages.  max_len: the longest one sequence may
        get (default: n_tokens).  max_step_tokens: the most tokens one sequence brings
        in one step (default: max_len); it sizes the rings of windowed groups.
        device None keeps the bookkeeping only (no storage), for tests on the host."""
        if n_slots <= 0 or n_tokens <= 0:
            raise CacheError("the cache needs at least one slot and one token")
        self.layout = layout
        self.n_slots = int(n_slots)
        self.n_pages = pages_for(n_tokens)
        self.max_len = int(max_len) if max_len else self.n_pages * PAGE
        self.max_step_tokens = int(max_step_tokens) if max_step_tokens else self.max_len
        self.dtype, self.device = dtype, device
        self.slots = FreeList(self.n_slots, "slot")
        self.lengths: List[int] = [0] * self.n_slots
        self.groups: List[KVGroup] = []
        self.group_of_run: Dict[int, Tuple[int, int]] = {}
        by_spec: Dict[KVSpec, List[int]] = {}
        for run in sorted(layout.kv):
            by_spec.setdefault(layout.kv[run], []).append(run)
        width = min(self.n_pages, pages_for(self.max_len))
        for spec, runs in by_spec.items():
            if spec.window is None:
                ring, n_pages = width, self.n_pages
            else:
                ring = min(width, pages_for(spec.window + self.max_step_tokens - 1) + 1)
                n_pages = min(self.n_pages, self.n_slots * ring)
            g = KVGroup(len(self.groups), spec, runs, n_pages, ring, min(width, ring))
            for i, run in enumerate(runs):
                self.group_of_run[run] = (g.index, i)
            self.groups.append(g)
        self.states = {}
        self._arena = self._arena_table = None
        if device is not None:
            import torch
            for g in self.groups:
                shape = (len(g.runs), g.n_pages, g.spec.n_kv_heads, PAGE, g.spec.head_dim)
                g.k = torch.empty(shape, dtype=dtype, device=device)
                g.v = torch.empty(shape, dtype=dtype, device=device)
            # all fixed-size state lies in one arena, region after region (each [slots, row]), so that one
            # kernel launch zeroes a slot's row of every state when the slot opens
            regions, off = [], 0
            for name, (shape, dt) in layout.states.items():
                td = getattr(torch, dt)
                n = 1
                for d in shape:
                    n *= int(d)
                row = n * torch.empty((), dtype=td).element_size()
                if row % 4:
                    raise CacheError(f"state {name}: a sequence's share ({row} bytes) must be a multiple of 4 bytes")
                regions.append((name, tuple(shape), td, off, row))
                off += (self.n_slots * row + 255) // 256 * 256
            self._arena = torch.zeros(max(off, 256), dtype=torch.uint8, device=device)
            for name, shape, td, at, row in regions:
                self.states[name] = self._arena[at:at + self.n_slots * row].view(td).view((self.n_slots,) + shape)
            if regions and torch.device(device).type == "cuda":
                self._arena_table = torch.tensor([[at, row] for _, _, _, at, row in regions], dtype=torch.int64, device=device)

    # ------------------------------------------------------------ sequences
    def open(self) -> int:
        """Takes a free slot for a new, empty sequence and zeroes its fixed-size state."""
        (slot,) = self.slots.take(1)
        self.lengths[slot] = 0
        for g in self.groups:
            g.tables[slot] = []
        if self._arena_table is not None:
            from .. import kernels
            kernels.zero_rows(self._arena, self._arena_table, slot)
        else:
            for t in self.states.values():
                t[slot].zero_()
        return slot

    def close(self, slot: int) -> None:
        """Gives back the slot and everything it holds."""
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is not open (closed twice?)")
        for g in self.groups:
            g.pool.give_back(g.tables.pop(slot))
        self.lengths[slot] = 0
        self.slots.give_back([slot])

    def length(self, slot: int) -> int:
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is not open")
        return self.lengths[slot]

    def reserve(self, slots: Sequence[int], new_tokens: Sequence[int]) -> None:
        """Makes room for new_tokens[i] more positions in slots[i], for all of them or,
        if slots or pages run out, for none (CacheFull)."""
        need = [0] * len(self.groups)
        for s, n in zip(slots, new_tokens):
            if not self.slots.is_held(s):
                raise CacheError(f"slot {s} is not open")
            if n <= 0:
                raise CacheError(f"slot {s}: a step must bring at least one token")
            if n > self.max_step_tokens:
                raise CacheFull(f"slot {s}: {n} tokens in one step, the cache was sized for {self.max_step_tokens}")
            total = self.lengths[s] + n
            if total > self.max_len:
                raise CacheFull(f"slot {s}: {total} positions exceed the longest sequence allowed ({self.max_len})")
            for g in self.groups:
                need[g.index] += g.pages_needed(total) - len(g.tables[s])
        if len(set(slots)) != len(slots):
            raise CacheError(f"slots {list(slots)} name one twice")
        for g in self.groups:
            if need[g.index] > g.pool.free_count:
                raise CacheFull(f"group {g.index}: need {need[g.index]} more pages, {g.pool.free_count} of "
                                f"{g.n_pages} are free")
        for s, n in zip(slots, new_tokens):
            total = self.lengths[s] + n
            for g in self.groups:
                g.tables[s].extend(g.pool.take(g.pages_needed(total) - len(g.tables[s])))

    def advance(self, slots: Sequence[int], new_tokens: Sequence[int]) -> None:
        for s, n in zip(slots, new_tokens):
            self.lengths[s] += n

    def table_rows(self, group: int, slots: Sequence[int], width: Optional[int] = None) -> List[List[int]]:
        """Page tables of these slots (slot -1: padding), padded with zeros to `width`
        entries (default: the group's full table width)."""
        g = self.groups[group]
        width = g.table_width if width is None else width
        rows = []
        for s in slots:
            t = g.tables[s] if s >= 0 else []
            if len(t) > width:
                raise CacheError(f"slot {s} holds {len(t)} pages of group {group}, the table has {width} entries")
            rows.append(t + [0] * (width - len(t)))
        return rows

    # ---------------------------------------------------------------- checks
    def tokens_held(self) -> int:
        """Positions held by live sequences in whole pages (the widest group counts)."""
        return max((g.pool.held_count for g in self.groups), default=0) * PAGE

    def check(self) -> None:
        """Nothing lost, held twice or freed twice: used by tests after every move."""
        self.slots.check()
        for g in self.groups:
            g.pool.check()
            seen = set()
            for s, pages in g.tables.items():
                assert self.slots.is_held(s), f"group {g.index} has a table for closed slot {s}"
                for p in pages:
                    assert g.pool.is_held(p), f"slot {s} lists page {p} that the pool thinks free"
                    assert p not in seen, f"page {p} of group {g.index} is in two tables"
                    seen.add(p)
                # a reservation made for a step that has not been counted yet may hold more pages than the
                # length needs, never fewer and never more than the ring
                assert g.pages_needed(self.lengths[s]) <= len(pages) <= g.ring_pages, \
                    f"slot {s} of length {self.lengths[s]} holds {len(pages)} pages of group {g.index}"
            assert len(seen) == g.pool.held_count, f"group {g.index}: {g.pool.held_count - len(seen)} pages are lost"

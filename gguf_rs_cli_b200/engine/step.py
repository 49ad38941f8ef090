"""The step function: a batch of sequences, each bringing its next tokens (a whole
prompt, a further piece of one, or one token), run as one packed batch from the
cache; returns the logits at the wanted places.

The reference's step is one token of one sequence (`forward_cpu(token, pos, cache)`,
src/model/llama.rs:343) and its prompt loop calls it once per token
(src/main.rs:241-256); this one takes all tokens of all sequences at once.  A token's
position is its index in its sequence, for the cache and for the rotation alike
(src/model/llama.rs:370-373).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

from .. import native
from ..cache.cache import Cache
from ..kernels import check_tc_status
from ..models.decoder import Decoder
from ..parts.base import HostBatch, StepContext, Workspace

SAMPLER_STATES = {"sampler.recent": ((64,), "int32"), "sampler.count": ((), "int32")}


class StepError(ValueError):
    """A step that cannot run: bad slot, bad token id, empty entry; nothing was launched."""


@dataclass
class Entry:
    """One sequence's share of a step: its slot, its next tokens, and the places among
    these tokens whose logits are wanted."""
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


class Engine:
    def __init__(self, model: Decoder, n_tokens: int, n_slots: int, max_len: Optional[int] = None,
                 max_step_tokens: Optional[int] = None):
        """n_tokens: the most positions that live sequences hold together, each rounded up
        to whole pages of 64.  n_slots: the most live sequences.  max_len: the longest
        sequence (default: the model's max position, at most n_tokens)."""
        native.require_device()
        self.model, self.device, self.dtype = model, model.device, model.dtype
        layout = model.cache_layout()
        layout.states.update(SAMPLER_STATES)
        if max_len is None:
            max_len = model.spec.max_position
        self.cache = Cache(layout, n_slots, n_tokens, max_len=min(int(max_len), ((n_tokens + 63) // 64) * 64),
                           max_step_tokens=max_step_tokens, dtype=self.dtype, device=self.device)
        self.ws = Workspace(self.device)
        self.runs = model.run_views(self.cache)
        self.vocab_size = model.spec.vocab_size
        self._meta_ring = None
        self._meta_slot = None
        self.launches = 0

    # ------------------------------------------------------------ sequences
    def open(self) -> int:
        return self.cache.open()

    def close(self, slot: int) -> None:
        self.cache.close(slot)

    def check(self) -> None:
        """After a synchronise: raises if a kernel's bounded wait gave up during the steps
        since the last check."""
        check_tc_status()

    # ----------------------------------------------------------------- plan
    def _meta(self, n: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """Pinned host and device buffers for a step's index arrays.  Steps do not wait for
        one another on the host, so the staging buffers form a ring, and one is written
        again only after the copy that last read it has run."""
        if self._meta_ring is None or self._meta_ring[0][0].numel() < n:
            size = max(n, 4096)
            self._meta_ring = [(torch.empty(size, dtype=torch.int32, pin_memory=True),
                                torch.empty(size, dtype=torch.int32, device=self.device)) for _ in range(4)]
            self._meta_events = [None] * 4
            self._meta_next = 0
        i = self._meta_next
        self._meta_next = (i + 1) % len(self._meta_ring)
        if self._meta_events[i] is not None:
            self._meta_events[i].synchronize()
        self._meta_slot = i
        return self._meta_ring[i]

    PLAN_WORDS = 4096

    def meta_size(self, batch: int) -> int:
        """int32 words of index arrays for a padded batch of single tokens with full tables, and room for
        what parts plan for such a step."""
        return 8 * batch + 1 + batch * sum(g.table_width for g in self.cache.groups) + self.PLAN_WORDS

    def plan(self, entries: Sequence[Entry], pad_to: Optional[int] = None, full_tables: bool = False,
             want_all: bool = False, meta: Optional[Tuple[torch.Tensor, torch.Tensor]] = None
             ) -> Tuple[StepContext, torch.Tensor, int]:
        """Checks the entries, reserves cache room and ships the step's index arrays to the
        device in one copy.  pad_to pads a batch of single tokens with entries that change
        nothing; full_tables, want_all (every row, padding too) and meta (pinned host and
        device buffers to use) give the arrays the same layout and addresses every step, as
        a captured graph needs.  Returns (context, wanted rows, number of wanted rows)."""
        if not entries:
            raise StepError("a step needs at least one entry")
        V = self.vocab_size
        slots, qlens = [], []
        for e in entries:
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"slot {e.slot}: an entry must bring at least one token")
            for t in e.tokens:
                if not 0 <= int(t) < V:
                    raise StepError(f"slot {e.slot}: token id {t} is outside the vocabulary (0..{V - 1})")
            for w in e.want:
                if not 0 <= int(w) < n:
                    raise StepError(f"slot {e.slot}: wanted place {w} is not among its {n} tokens")
            slots.append(int(e.slot))
            qlens.append(n)
        starts = [self.cache.length(s) for s in slots]
        self.cache.reserve(slots, qlens)

        B, T = len(entries), sum(qlens)
        Bp, Tp = B, T
        if pad_to is not None and pad_to > B:
            if max(qlens) != 1:
                raise StepError("only steps of single tokens can be padded")
            Bp = Tp = pad_to
        tokens, seq_of, pos, cu, want = [], [], [], [0], []
        for b, e in enumerate(entries):
            tokens += [int(t) for t in e.tokens]
            seq_of += [b] * qlens[b]
            pos += list(range(starts[b], starts[b] + qlens[b]))
            want += [cu[-1] + int(w) for w in e.want]
            cu.append(cu[-1] + qlens[b])
        padT, padB = Tp - T, Bp - B
        tokens += [0] * padT
        seq_of += [-1] * padT
        pos += [0] * padT
        cu += [cu[-1]] * padB
        slots_p = slots + [-1] * padB
        starts_p = starts + [0] * padB
        qlens_p = qlens + [0] * padB
        if want_all:
            want = list(range(Tp))
        flat = tokens + seq_of + pos + slots_p + starts_p + qlens_p + cu + want
        offs, o = {}, 0
        for name, n in (("tokens", Tp), ("seq_of", Tp), ("pos", Tp), ("slots", Bp), ("starts", Bp), ("qlens", Bp),
                        ("cu", Bp + 1), ("want", len(want))):
            offs[name] = (o, n)
            o += n
        max_kv = max(s + q for s, q in zip(starts, qlens))
        # index arrays that parts lay out for themselves travel in the same copy
        batch = HostBatch(slots, starts, qlens, decode=max(qlens) == 1, max_qlen=max(qlens), max_kv=max_kv)
        plan_offs = []
        for key, part in self.model.planners:
            for name, values in part.plan(batch).items():
                values = [int(v) for v in values]
                plan_offs.append((key, name, len(flat), len(values)))
                flat += values
        table_offs = []
        for g in self.cache.groups:
            # only as many table entries as this step's longest sequence uses, unless the
            # caller needs the same layout every step (a captured graph)
            width = g.table_width if full_tables else max(1, g.pages_needed(max_kv))
            rows = self.cache.table_rows(g.index, slots_p, width)
            table_offs.append((len(flat), Bp, width))
            for r in rows:
                flat += r
        own = meta is None
        host, dev = self._meta(len(flat)) if own else meta
        if len(flat) > host.numel():
            raise StepError(f"the step's index arrays ({len(flat)} words) exceed the buffer given ({host.numel()})")
        host[:len(flat)] = torch.tensor(flat, dtype=torch.int32)
        dev[:len(flat)].copy_(host[:len(flat)], non_blocking=True)
        if own:
            ev = torch.cuda.Event()
            ev.record()
            self._meta_events[self._meta_slot] = ev

        def view(name):
            a, n = offs[name]
            return dev[a:a + n]

        ctx = StepContext(
            T=Tp, B=Bp, dtype=self.dtype, tokens=view("tokens"), seq_of=view("seq_of"), pos=view("pos"),
            slots=view("slots"), starts=view("starts"), qlens=view("qlens"), cu=view("cu"),
            tables=[dev[a:a + b * w].view(b, w) for a, b, w in table_offs], cache=self.cache, ws=self.ws,
            decode=max(qlens) == 1, max_qlen=max(qlens), max_kv=max_kv,
            host={"slots": slots, "starts": starts, "qlens": qlens, "h2d_bytes": 4 * len(flat), "layout": offs,
                  "table_offs": table_offs, "n_words": len(flat), "batch": batch,
                  "plan_words": sum(n for _, _, _, n in plan_offs)})
        for key, name, a, n in plan_offs:
            ctx.plans.setdefault(key, {})[name] = dev[a:a + n]
        return ctx, view("want"), len(want)

    # ----------------------------------------------------------------- step
    def step(self, entries: Sequence[Entry]) -> Optional[torch.Tensor]:
        """Runs the entries' tokens as one batch from the cache and advances the sequences.
        Returns float32 logits [wanted, V] in the order of the entries and of each `want`
        (None when nothing is wanted; the tokens still enter the cache).

        The tensor returned is one of the engine's own buffers (a step allocates nothing): a later
        step that wants the same number of rows writes over it.  Copy what has to outlive the next
        step (`.clone()`, or `.cpu()` as the replay program does)."""
        entries = [e if isinstance(e, Entry) else Entry(*e) for e in entries]
        ctx, want_rows, n_want = self.plan(entries)
        logits = self.model.forward(ctx, self.runs, want_rows)
        self.cache.advance(ctx.host["slots"], ctx.host["qlens"])
        return logits if n_want else None

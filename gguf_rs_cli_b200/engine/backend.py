"""The generation loop's backend on the device: engine step + sampler."""
from __future__ import annotations

from typing import List, Optional, Sequence

import sys

import numpy as np
import torch

from ..cache.pool import PAGE, CacheFull, pages_for
from ..parts.base import HostBatch
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .step import Engine, Entry, StepError


class DecodeGraph:
    """One captured decode step (model + sampling) for a padded batch size and one set of
    sampling options.  Its index arrays live in buffers of its own, so replaying it needs
    one host-to-device copy and one graph launch."""

    def __init__(self, engine: Engine, bucket: int):
        self.bucket = bucket
        n = engine.meta_size(bucket)
        self.meta = (torch.empty(n, dtype=torch.int32).pin_memory(), torch.empty(n, dtype=torch.int32, device=engine.device))
        self.keys_host = torch.zeros(bucket, dtype=torch.int64).pin_memory()
        self.keys_dev = torch.zeros(bucket, dtype=torch.int64, device=engine.device)
        self.out_dev = torch.zeros(bucket, dtype=torch.int32, device=engine.device)
        self.graph = None
        self.warm = False
        self.launches = 0
        # what the host buffer holds, for steps that only move on by one token: the batch it was laid out for,
        # where each array lies, and a numpy view of the pinned buffer
        self.laid_out_for = None
        self.keys = None
        self.layout = None
        self.table_offs = None
        self.n_words = 0
        self.plan_words = 0          # words that parts planned for the step: such a graph is laid out anew every step
        self.host_np = self.meta[0].numpy()
        self.copied = None           # passed when the last copy out of the pinned buffer has run: then it may be written again


class Pending:
    """A step that has been launched: its sampled tokens are in `out_host` once `event` has passed.  `out_dev`
    holds them on the device, where the step after may take them from (EngineBackend.begin_after)."""
    __slots__ = ("slots", "keys", "params", "n", "out_dev", "out_host", "event", "marks", "n_tokens")

    def __init__(self, slots, keys, params, out_dev, out_host, event):
        self.slots, self.keys, self.params, self.n = list(slots), list(keys), params, len(slots)
        self.out_dev, self.out_host, self.event = out_dev, out_host, event
        self.marks, self.n_tokens = None, 0


def format_marks(marks, n_tokens: int) -> str:
    """One line per profiled step, stage by stage, in the manner of the reference's
    `[ts0-1: 0.02ms] ... [total GPU: 1.23ms]` (src/gpu/mod.rs:345-361), with the stages' names."""
    parts = [f"[{marks[i][0]}: {marks[i - 1][1].elapsed_time(marks[i][1]):.3f}ms]" for i in range(1, len(marks))]
    total = marks[0][1].elapsed_time(marks[-1][1]) if len(marks) > 1 else 0.0
    return f"[GPU step of {n_tokens} tokens] " + " ".join(parts) + f" [total GPU: {total:.3f}ms]"


def bucket_of(n: int) -> int:
    b = 1
    while b < n:
        b *= 2
    return b


class EngineBackend:
    def __init__(self, engine: Engine, use_graphs: bool = True):
        """use_graphs: decode steps run as captured CUDA graphs where every part of the model allows it
        (`graph_class`).  profile: every step runs eagerly with a time stamp after each stage and one line
        per step goes to `profile_out` (the reference's --debug-gpu, src/gpu/mod.rs:345-361)."""
        self.engine = engine
        self.use_graphs = use_graphs
        self.profile = False
        self.profile_out = sys.stderr
        self._graphs = {}
        self._batch = None           # (slots of the last decode step, their lengths after it)
        self._last_graph = None
        self.sampler = Sampler(engine.cache, engine.device)
        self.context_limit = engine.cache.max_len
        n = engine.cache.n_slots
        self._out_dev = torch.zeros(n, dtype=torch.int32, device=engine.device)
        # two steps may be in flight (the one whose tokens the host waits for and the one launched ahead of it)
        self._out_hosts = [torch.zeros(n, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._events = [torch.cuda.Event() for _ in range(2)]
        self._turn = 0
        self._keys_host = torch.zeros(n, dtype=torch.int64).pin_memory()
        self._keys_dev = torch.zeros(n, dtype=torch.int64, device=engine.device)
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.steps_ahead = 0         # steps launched before the tokens of the step in front of them were read
        self._ones = [1] * n

    def admit(self, prompt_lens: Sequence[int], max_new: int) -> int:
        """Prompts are admitted in order while slots and pages last, counting each at the
        length it may reach."""
        cache = self.engine.cache
        free_pages = min(g.pool.free_count for g in cache.groups) if cache.groups else 1 << 30
        free_slots = cache.slots.free_count
        n = 0
        for plen in prompt_lens:
            need = pages_for(min(plen + max_new, cache.max_len))
            if n >= free_slots or need > free_pages:
                break
            free_pages -= need
            n += 1
        return n

    def open(self) -> int:
        self._batch = self._last_graph = None
        return self.engine.open()

    def close(self, slot: int) -> None:
        self._batch = self._last_graph = None
        self.engine.close(slot)

    def _pending(self, slots, keys, params, out_dev) -> Pending:
        """Asks for the step's tokens on the host and marks the place in the stream where they are there."""
        i = self._turn
        self._turn = 1 - i
        n = len(slots)
        self._out_hosts[i][:n].copy_(out_dev[:n], non_blocking=True)
        self._events[i].record()
        self.d2h_bytes += 4 * n
        return Pending(slots, keys, params, out_dev, self._out_hosts[i], self._events[i])

    def _launch_decode_graph(self, slots, tokens, keys, params, after: Optional[Pending] = None) -> Optional[Pending]:
        """A step of single tokens through a captured graph: the first call of a batch size
        runs the same kernels eagerly (and sizes every buffer), the second captures.  While the
        same sequences go on token by token, the index arrays are updated in place in the pinned
        buffer (tokens, positions, and a table entry when a sequence enters a new page) instead of
        being laid out again.  tokens None: each sequence is fed what the step `after` sampled for it,
        on the device, so that this step can be launched before the host has seen those tokens."""
        from .. import native
        eng, n = self.engine, len(slots)
        cache = eng.cache
        slots_t = tuple(slots)
        if self._batch is not None and self._batch[0] == slots_t:
            lengths = self._batch[1]
        else:
            lengths = np.array([cache.length(s) for s in slots], dtype=np.int64)
        # what a captured graph fixes (grids that depend on the lengths, a part's host-side choices) is the
        # parts' to say: one graph per class of step
        longest = int(lengths.max())
        cls = eng.model.graph_class(HostBatch(slots, lengths, self._ones[:n], decode=True, max_qlen=1, max_kv=longest + 1))
        if cls is None:
            return None
        key = (bucket_of(n), cls, params.temperature, params.top_k, params.top_p, params.rep_penalty)
        dg = self._graphs.get(key)
        if dg is None:
            dg = self._graphs[key] = DecodeGraph(eng, key[0])
        if dg.copied is not None:
            dg.copied.synchronize()
        if (dg.graph is not None and self._last_graph is dg and dg.laid_out_for == slots_t and dg.keys == keys
                and dg.plan_words == 0):
            self._advance_in_place(dg, slots, tokens, lengths)
            self._feed_from(dg, after, n)
            dg.graph.replay()
            native.count_launches(dg.launches)
            h2d = 4 * dg.n_words
        else:
            feed = [0] * n if tokens is None else tokens
            entries = [Entry(s, (int(t),), (0,)) for s, t in zip(slots, feed)]
            ctx, want_rows, _ = eng.plan(entries, pad_to=dg.bucket, full_tables=True, want_all=True, meta=dg.meta)
            dg.laid_out_for, dg.layout = slots_t, ctx.host["layout"]
            dg.table_offs, dg.n_words = ctx.host["table_offs"], ctx.host["n_words"]
            if dg.graph is not None and ctx.host["plan_words"] != dg.plan_words:
                raise StepError("a part planned index arrays of another size than in the step its graph was captured "
                                "from: its graph_class must tell such steps apart")
            dg.plan_words = ctx.host["plan_words"]
            dg.keys = list(keys)
            dg.keys_host[:n] = torch.tensor(keys, dtype=torch.int64)
            dg.keys_dev.copy_(dg.keys_host, non_blocking=True)
            self._copied(dg)
            self._feed_from(dg, after, n)

            def body():
                logits = eng.model.forward(ctx, eng.runs, want_rows)
                self.sampler.sample(logits, ctx.slots, dg.keys_dev, params, dg.out_dev)

            if dg.graph is None and dg.warm:
                torch.cuda.current_stream().synchronize()
                before = native.launch_count()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    body()
                dg.graph, dg.launches = g, native.launch_count() - before
            if dg.graph is not None:
                dg.graph.replay()
                native.count_launches(dg.launches)
            else:
                body()
                dg.warm = True
            cache.advance(slots, [1] * n)
            h2d = ctx.host["h2d_bytes"] + 8 * dg.bucket
        self._batch, self._last_graph = (slots_t, lengths + 1), dg
        self.h2d_bytes += h2d
        return self._pending(slots, keys, params, dg.out_dev)

    def _copied(self, dg: DecodeGraph) -> None:
        if dg.copied is None:
            dg.copied = torch.cuda.Event()
        dg.copied.record()

    def _feed_from(self, dg: DecodeGraph, after: Optional[Pending], n: int) -> None:
        """The tokens of the step that is being launched are the ones `after` sampled: copied on the device,
        behind the copy of the index arrays and before the graph."""
        if after is not None:
            a, _ = dg.layout["tokens"]
            dg.meta[1][a:a + n].copy_(after.out_dev[:n], non_blocking=True)

    def _advance_in_place(self, dg: DecodeGraph, slots, tokens: np.ndarray, lengths: np.ndarray) -> None:
        """The same batch one token further: checks, cache room, and the few words that change."""
        eng, cache, n = self.engine, self.engine.cache, len(slots)
        if tokens is not None and (tokens.min() < 0 or tokens.max() >= eng.vocab_size):
            raise StepError(f"a token id of {tokens.tolist()} is outside the vocabulary (0..{eng.vocab_size - 1})")
        if int(lengths.max()) + 1 > cache.max_len:
            raise CacheFull(f"a sequence would exceed the longest sequence allowed ({cache.max_len})")
        fresh = np.nonzero(lengths % PAGE == 0)[0]               # these enter a new page (where their group still grows)
        if fresh.size:
            cache.reserve([slots[b] for b in fresh], [1] * fresh.size)
            for g, (at, _, width) in zip(cache.groups, dg.table_offs):
                for b in fresh:
                    row = g.tables[slots[b]]
                    dg.host_np[at + b * width:at + b * width + len(row)] = row
        h = dg.host_np
        if tokens is not None:
            a, _ = dg.layout["tokens"]
            h[a:a + n] = tokens
        a, _ = dg.layout["pos"]
        h[a:a + n] = lengths
        a, _ = dg.layout["starts"]
        h[a:a + n] = lengths
        dg.meta[1][:dg.n_words].copy_(dg.meta[0][:dg.n_words], non_blocking=True)
        self._copied(dg)
        for s in slots:
            cache.lengths[s] += 1

    def begin(self, slots: List[int], feeds: List[List[int]], keys: List[int], params: SamplingParams) -> Pending:
        """Launches a step (each sequence's next tokens, one sampled token per sequence) and returns without
        waiting for it."""
        if self.use_graphs and not self.profile and all(len(f) == 1 for f in feeds):
            tokens = np.fromiter((f[0] for f in feeds), dtype=np.int64, count=len(feeds))
            pending = self._launch_decode_graph(slots, tokens, keys, params)
            if pending is not None:
                return pending
        eng, n = self.engine, len(slots)
        self._batch = self._last_graph = None
        entries = [Entry(s, f, (len(f) - 1,)) for s, f in zip(slots, feeds)]
        self._keys_host[:n] = torch.tensor(keys, dtype=torch.int64)
        self._keys_dev[:n].copy_(self._keys_host[:n], non_blocking=True)
        ctx, want_rows, n_want = eng.plan(entries)
        if self.profile:
            ctx.marks = []
            ctx.mark("start")
        logits = eng.model.forward(ctx, eng.runs, want_rows)
        eng.cache.advance(ctx.host["slots"], ctx.host["qlens"])
        self.sampler.sample(logits, ctx.slots[:n], self._keys_dev[:n], params, self._out_dev)
        ctx.mark("sample")
        self.h2d_bytes += ctx.host["h2d_bytes"] + 8 * n
        pending = self._pending(slots, keys, params, self._out_dev)
        if self.profile:
            pending.marks, pending.n_tokens = ctx.marks, ctx.T
        return pending

    def begin_after(self, pending: Pending) -> Optional[Pending]:
        """Launches the step after `pending` for the same sequences, each fed the token that `pending` samples
        for it, before the host has seen those tokens: the device does not wait for the host between two steps.
        None where that is not possible (steps that are not captured); then the caller finishes `pending` and
        begins the next step with the tokens in hand.  A caller that then finds a sequence ended by its token
        drops that sequence's token of the step launched here."""
        if not (self.use_graphs and not self.profile):
            return None
        ahead = self._launch_decode_graph(pending.slots, None, pending.keys, pending.params, after=pending)
        if ahead is not None:
            self.steps_ahead += 1
        return ahead

    def finish(self, pending: Pending) -> List[int]:
        """Waits for a step launched by begin or begin_after and returns its sampled tokens."""
        pending.event.synchronize()
        if pending.marks is not None:
            print(format_marks(pending.marks, pending.n_tokens), file=self.profile_out, flush=True)
        self.engine.check()
        return pending.out_host[:pending.n].tolist()

    def run(self, slots: List[int], feeds: List[List[int]], keys: List[int], params: SamplingParams) -> List[int]:
        return self.finish(self.begin(slots, feeds, keys, params))

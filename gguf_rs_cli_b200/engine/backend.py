"""The generation loop's backend on the device: engine step + sampler."""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch

from .. import kernels
from ..cache.pool import PAGE, CacheFull, pages_for
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
        self.host_np = self.meta[0].numpy()


def bucket_of(n: int) -> int:
    b = 1
    while b < n:
        b *= 2
    return b


class EngineBackend:
    def __init__(self, engine: Engine, use_graphs: bool = True):
        self.engine = engine
        self.use_graphs = use_graphs
        self._graphs = {}
        self._batch = None           # (slots of the last decode step, their lengths after it)
        self._last_graph = None
        self.sampler = Sampler(engine.cache, engine.device)
        self.context_limit = engine.cache.max_len
        n = engine.cache.n_slots
        self._out_dev = torch.zeros(n, dtype=torch.int32, device=engine.device)
        self._out_host = torch.zeros(n, dtype=torch.int32).pin_memory()
        self._keys_host = torch.zeros(n, dtype=torch.int64).pin_memory()
        self._keys_dev = torch.zeros(n, dtype=torch.int64, device=engine.device)
        self.h2d_bytes = 0
        self.d2h_bytes = 0

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

    def _run_decode_graph(self, slots, feeds, keys, params) -> List[int]:
        """A step of single tokens through a captured graph: the first call of a batch size
        runs the same kernels eagerly (and sizes every buffer), the second captures.  While the
        same sequences go on token by token, the index arrays are updated in place in the pinned
        buffer (tokens, positions, and a table entry when a sequence enters a new page) instead of
        being laid out again."""
        from .. import native
        eng, n = self.engine, len(slots)
        cache = eng.cache
        slots_t = tuple(slots)
        if self._batch is not None and self._batch[0] == slots_t:
            lengths = self._batch[1]
        else:
            lengths = np.array([cache.length(s) for s in slots], dtype=np.int64)
        # the attention kernels' page splits are fixed in a captured graph: one graph per class of length
        key = (bucket_of(n), kernels.decode_split_class(int(lengths.max()) + 1), params.temperature, params.top_k,
               params.top_p, params.rep_penalty)
        dg = self._graphs.get(key)
        if dg is None:
            dg = self._graphs[key] = DecodeGraph(eng, key[0])
        tokens = np.fromiter((f[0] for f in feeds), dtype=np.int64, count=n)
        if dg.graph is not None and self._last_graph is dg and dg.laid_out_for == slots_t and dg.keys == keys:
            self._advance_in_place(dg, slots, tokens, lengths)
            dg.graph.replay()
            native.count_launches(dg.launches)
            h2d = 4 * dg.n_words
        else:
            entries = [Entry(s, (int(t),), (0,)) for s, t in zip(slots, tokens)]
            ctx, want_rows, _ = eng.plan(entries, pad_to=dg.bucket, full_tables=True, want_all=True, meta=dg.meta)
            dg.laid_out_for, dg.layout = slots_t, ctx.host["layout"]
            dg.table_offs, dg.n_words = ctx.host["table_offs"], ctx.host["n_words"]
            dg.keys = list(keys)
            dg.keys_host[:n] = torch.tensor(keys, dtype=torch.int64)
            dg.keys_dev.copy_(dg.keys_host, non_blocking=True)

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
        self._out_host[:n].copy_(dg.out_dev[:n], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        eng.check()
        self.h2d_bytes += h2d
        self.d2h_bytes += 4 * n
        return self._out_host[:n].tolist()

    def _advance_in_place(self, dg: DecodeGraph, slots, tokens: np.ndarray, lengths: np.ndarray) -> None:
        """The same batch one token further: checks, cache room, and the few words that change."""
        eng, cache, n = self.engine, self.engine.cache, len(slots)
        if tokens.min() < 0 or tokens.max() >= eng.vocab_size:
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
        a, _ = dg.layout["tokens"]
        h[a:a + n] = tokens
        a, _ = dg.layout["pos"]
        h[a:a + n] = lengths
        a, _ = dg.layout["starts"]
        h[a:a + n] = lengths
        dg.meta[1][:dg.n_words].copy_(dg.meta[0][:dg.n_words], non_blocking=True)
        for s in slots:
            cache.lengths[s] += 1

    def run(self, slots: List[int], feeds: List[List[int]], keys: List[int], params: SamplingParams) -> List[int]:
        if self.use_graphs and all(len(f) == 1 for f in feeds):
            return self._run_decode_graph(slots, feeds, keys, params)
        eng, n = self.engine, len(slots)
        self._batch = self._last_graph = None
        entries = [Entry(s, f, (len(f) - 1,)) for s, f in zip(slots, feeds)]
        self._keys_host[:n] = torch.tensor(keys, dtype=torch.int64)
        self._keys_dev[:n].copy_(self._keys_host[:n], non_blocking=True)
        ctx, want_rows, n_want = eng.plan(entries)
        logits = eng.model.forward(ctx, eng.runs, want_rows)
        eng.cache.advance(ctx.host["slots"], ctx.host["qlens"])
        self.sampler.sample(logits, ctx.slots[:n], self._keys_dev[:n], params, self._out_dev)
        self._out_host[:n].copy_(self._out_dev[:n], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        eng.check()
        self.h2d_bytes += ctx.host["h2d_bytes"] + 8 * n
        self.d2h_bytes += 4 * n
        return self._out_host[:n].tolist()

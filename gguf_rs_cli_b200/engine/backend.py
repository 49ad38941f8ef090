"""The generation loop's backend on the device: engine step + sampler."""
from __future__ import annotations

from typing import List, Sequence

import torch

from .. import kernels
from ..cache.pool import pages_for
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .step import Engine, Entry


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
        return self.engine.open()

    def close(self, slot: int) -> None:
        self.engine.close(slot)

    def _run_decode_graph(self, slots, feeds, keys, params) -> List[int]:
        """A step of single tokens through a captured graph: the first call of a batch size
        runs the same kernels eagerly (and sizes every buffer), the second captures."""
        from .. import native
        eng, n = self.engine, len(slots)
        # the attention kernels' page splits are fixed in a captured graph: one graph per class of length
        longest = max(eng.cache.length(s) for s in slots) + 1
        key = (bucket_of(n), kernels.decode_split_class(longest), params.temperature, params.top_k, params.top_p,
               params.rep_penalty)
        dg = self._graphs.get(key)
        if dg is None:
            dg = self._graphs[key] = DecodeGraph(eng, key[0])
        entries = [Entry(s, f, (0,)) for s, f in zip(slots, feeds)]
        ctx, want_rows, _ = eng.plan(entries, pad_to=dg.bucket, full_tables=True, want_all=True, meta=dg.meta)
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
        eng.cache.advance(ctx.host["slots"], ctx.host["qlens"])
        self._out_host[:n].copy_(dg.out_dev[:n], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        eng.check()
        self.h2d_bytes += ctx.host["h2d_bytes"] + 8 * dg.bucket
        self.d2h_bytes += 4 * n
        return self._out_host[:n].tolist()

    def run(self, slots: List[int], feeds: List[List[int]], keys: List[int], params: SamplingParams) -> List[int]:
        if self.use_graphs and all(len(f) == 1 for f in feeds):
            return self._run_decode_graph(slots, feeds, keys, params)
        eng, n = self.engine, len(slots)
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

"""The generation loop's backend on the device: engine step + sampler."""
from __future__ import annotations

from typing import List, Sequence

import torch

from ..cache.pool import pages_for
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .step import Engine, Entry


class EngineBackend:
    def __init__(self, engine: Engine):
        self.engine = engine
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

    def run(self, slots: List[int], feeds: List[List[int]], keys: List[int], params: SamplingParams) -> List[int]:
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

"""The generation loop above the step function: batches of unequal prompts, stop
tokens, sequences that end earlier than their batch, and as many batches one after
another as there are requests.

Per sequence it decides in the reference's order (src/main.rs:279-311): sample from
the last logits; a stop token ends the sequence and is not emitted; then the count
limit; then the context limit (position >= context - 1); else the token is emitted
and fed back.  The loop itself touches no device: it drives a backend (`open`,
`close`, `run`, `admit`), so its decisions are tested on the host with a scripted one.

A backend that can launch a step without waiting for it (`begin`, `begin_after`,
`finish`) is driven one step ahead: while no sequence of the batch can end by a limit,
the next step is launched, fed on the device with the tokens of the step in flight,
before those tokens are read.  A stop token is then found one step late: the sequence's
row of the step that ran ahead is dropped, and its slot, already given back, is used by
nobody before that step has run, because everything runs in one stream.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

from ..sampling.params import SamplingParams, stream_key


class GenerationError(ValueError):
    """A request that cannot be run (empty prompt, prompt longer than the context)."""


@dataclass
class _Live:
    request: int
    slot: Optional[int]
    feed: List[int]
    pos: int = 0


class _StepByStep:
    """A backend that only has `run`, as one that launches and finishes: every step is finished when it begins."""

    def __init__(self, backend):
        self.backend = backend

    def begin(self, slots, feeds, keys, params):
        return self.backend.run(slots, feeds, keys, params)

    def begin_after(self, pending):
        return None

    def finish(self, pending):
        return pending


@dataclass
class GenerationStats:
    """What --stats prints (src/main.rs:118-122): prompt tokens and time, generated
    tokens and time."""
    prompt_tokens: int = 0
    prefill_seconds: float = 0.0
    generated_tokens: int = 0
    decode_seconds: float = 0.0
    decode_steps: int = 0
    batches: int = 0
    step_batch_sizes: List[int] = field(default_factory=list)


def generate_ids(backend, prompts: Sequence[Sequence[int]], max_tokens: int, params: SamplingParams = SamplingParams(),
                 stop_token_ids: Sequence[int] = (), max_batch: Optional[int] = None,
                 on_token: Optional[Callable[[int, int], None]] = None,
                 stats: Optional[GenerationStats] = None, clock: Optional[Callable[[], float]] = None,
                 context_limit: Optional[int] = None) -> List[List[int]]:
    """Returns the generated ids of every prompt, in the order of the prompts.

    backend.context_limit      positions one sequence may hold (`context_limit` may lower it)
    backend.admit(lens, n)     how many of the next prompts (lengths `lens`) may start together
                               when each may grow by n tokens; at least 1 or an error
    backend.open() -> slot     backend.close(slot)
    backend.run(slots, feeds, keys, params) -> one sampled token per sequence
    """
    params.validate()
    stops = set(int(s) for s in stop_token_ids)
    ctx = backend.context_limit if context_limit is None else min(backend.context_limit, int(context_limit))
    for i, p in enumerate(prompts):
        if len(p) == 0:
            raise GenerationError(f"prompt {i} is empty: a request needs at least one token")
        if len(p) > ctx:
            raise GenerationError(f"prompt {i} has {len(p)} tokens, the cache holds {ctx} per sequence")
    results: List[List[int]] = [[] for _ in prompts]
    keys = [stream_key(params.seed, i) for i in range(len(prompts))]
    now = clock or (lambda: 0.0)
    steps = backend if hasattr(backend, "begin_after") else _StepByStep(backend)
    nxt = 0
    while nxt < len(prompts):
        window = prompts[nxt:nxt + max_batch] if max_batch else prompts[nxt:]
        n = backend.admit([len(p) for p in window], max_tokens)
        if n < 1:
            raise GenerationError(f"prompt {nxt} does not fit the cache even alone")
        live = []
        try:
            for i in range(nxt, nxt + n):
                live.append(_Live(i, backend.open(), list(prompts[i])))
            nxt += n
            if stats:
                stats.batches += 1
            first = True
            rows, counts = live, [len(s.feed) for s in live]
            t0 = now()
            pending = steps.begin([s.slot for s in rows], [s.feed for s in rows], [keys[s.request] for s in rows], params)
            while live:
                # The step after, before this one's tokens are read: only while its rows would be this step's rows,
                # so none may have ended already and none may end by a limit now; a stop token shows one step late.
                ahead = None
                if all(s.slot is not None for s in rows) and not any(
                        len(results[s.request]) >= max_tokens or s.pos + c >= ctx - 1 for s, c in zip(rows, counts)):
                    ahead = steps.begin_after(pending)
                sampled = steps.finish(pending)
                dt = now() - t0
                t0 = now()
                if stats:
                    stats.step_batch_sizes.append(len(live))
                    if first:
                        stats.prompt_tokens += sum(counts)
                        stats.prefill_seconds += dt
                    else:
                        stats.decode_steps += 1
                        stats.decode_seconds += dt
                first = False
                still = []
                for s, c, tok in zip(rows, counts, sampled):
                    if s.slot is None:                     # ended a step ago: this row ran ahead for nothing
                        continue
                    s.pos += c
                    tok = int(tok)
                    if tok in stops or len(results[s.request]) >= max_tokens or s.pos >= ctx - 1:
                        backend.close(s.slot)          # given back at once: the next batch may use it
                        s.slot = None
                        continue
                    results[s.request].append(tok)
                    if stats:
                        stats.generated_tokens += 1
                    if on_token:
                        on_token(s.request, tok)
                    s.feed = [tok]
                    still.append(s)
                live = still
                if ahead is not None:
                    pending, counts = ahead, [1] * len(rows)
                    if not live:
                        steps.finish(ahead)                # nobody is left to read it
                elif live:
                    rows, counts = live, [1] * len(live)
                    pending = steps.begin([s.slot for s in rows], [s.feed for s in rows], [keys[s.request] for s in rows], params)
        finally:
            # a step, a callback or the cache may raise: whatever the batch still holds is given back
            for s in live:
                if s.slot is not None:
                    backend.close(s.slot)
                    s.slot = None
    return results

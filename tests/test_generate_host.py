"""The generation loop's decisions, with a scripted backend in place of the device."""
import pytest

from gguf_rs_cli_b200.engine import GenerationError, GenerationStats, generate_ids
from gguf_rs_cli_b200.sampling import SamplingParams, stream_key


class Scripted:
    """Sequences "generate" prompt[0]+1, +2, ...; keeps a log of every call and a slot pool."""

    def __init__(self, n_slots=2, context_limit=100, admit_limit=None):
        self.free = list(range(n_slots))
        self.context_limit = context_limit
        self.admit_limit = admit_limit
        self.state = {}
        self.log = []
        self.held_max = 0

    def admit(self, lens, max_new):
        n = min(len(lens), len(self.free))
        return n if self.admit_limit is None else min(n, self.admit_limit)

    def open(self):
        s = self.free.pop(0)
        self.state[s] = None
        self.held_max = max(self.held_max, len(self.state))
        self.log.append(("open", s))
        return s

    def close(self, slot):
        assert slot in self.state, "closed twice"
        del self.state[slot]
        self.free.append(slot)
        self.free.sort()
        self.log.append(("close", slot))

    def run(self, slots, feeds, keys, params):
        self.log.append(("run", list(slots), [list(f) for f in feeds]))
        out = []
        for s, f in zip(slots, feeds):
            if self.state[s] is None:
                self.state[s] = [f[0], 0, len(f)]
            else:
                assert len(f) == 1, "after the prompt a sequence brings one token"
                self.state[s][2] += 1
            self.state[s][1] += 1
            out.append(self.state[s][0] + self.state[s][1])
        return out


def test_max_tokens_and_order_of_results():
    b = Scripted(n_slots=3)
    out = generate_ids(b, [[10, 1], [20], [30, 1, 1]], max_tokens=3)
    assert out == [[11, 12, 13], [21, 22, 23], [31, 32, 33]]
    runs = [e for e in b.log if e[0] == "run"]
    assert runs[0][2] == [[10, 1], [20], [30, 1, 1]]              # prompts in one step
    assert all(all(len(f) == 1 for f in r[2]) for r in runs[1:])   # then one token each
    assert len(runs) == 4 and not b.state


def test_stop_token_ends_early_and_is_not_emitted():
    b = Scripted(n_slots=2)
    out = generate_ids(b, [[10], [20]], max_tokens=5, stop_token_ids=[12])
    assert out == [[11], [21, 22, 23, 24, 25]]
    runs = [e for e in b.log if e[0] == "run"]
    assert runs[1][1] == [0, 1] and runs[2][1] == [1]             # the finished one left the batch
    i_close0 = b.log.index(("close", 0))
    assert i_close0 < b.log.index(runs[2])                         # and gave its slot back at once


def test_batches_follow_one_another_and_reuse_slots():
    b = Scripted(n_slots=2)
    prompts = [[10 * i] for i in range(1, 6)]
    stats = GenerationStats()
    out = generate_ids(b, prompts, max_tokens=2, stats=stats)
    assert out == [[10 * i + 1, 10 * i + 2] for i in range(1, 6)]
    assert stats.batches == 3 and b.held_max == 2 and not b.state
    opens = [e[1] for e in b.log if e[0] == "open"]
    assert opens == [0, 1, 0, 1, 0]
    assert stats.generated_tokens == 10 and stats.prompt_tokens == 5


def test_max_batch_limits_a_batch():
    b = Scripted(n_slots=4)
    stats = GenerationStats()
    generate_ids(b, [[1], [2], [3]], max_tokens=1, max_batch=2, stats=stats)
    assert stats.batches == 2 and b.held_max == 2


def test_context_limit_stops_as_the_reference_does():
    # position >= context - 1 ends the sequence after sampling (src/main.rs:284-286)
    b = Scripted(n_slots=1, context_limit=8)
    out = generate_ids(b, [[10, 0, 0, 0, 0]], max_tokens=50)
    assert out == [[11, 12]]          # cache reaches 7 positions, never context - 1
    with pytest.raises(GenerationError, match="holds 8"):
        generate_ids(Scripted(n_slots=1, context_limit=8), [[1] * 9], max_tokens=1)


def test_zero_max_tokens_and_errors():
    assert generate_ids(Scripted(), [[5]], max_tokens=0) == [[]]
    with pytest.raises(GenerationError, match="empty"):
        generate_ids(Scripted(), [[1], []], max_tokens=1)
    with pytest.raises(GenerationError, match="does not fit"):
        generate_ids(Scripted(admit_limit=0), [[1]], max_tokens=1)
    with pytest.raises(ValueError, match="top_p"):
        generate_ids(Scripted(), [[1]], 1, SamplingParams(top_p=0.0))


def test_a_failing_step_or_callback_gives_every_slot_back():
    class Failing(Scripted):
        def run(self, slots, feeds, keys, params):
            if len([e for e in self.log if e[0] == "run"]) == 2:
                raise RuntimeError("the device gave up")
            return super().run(slots, feeds, keys, params)

    b = Failing(n_slots=3)
    with pytest.raises(RuntimeError, match="gave up"):
        generate_ids(b, [[10], [20], [30]], max_tokens=5, stop_token_ids=[21])       # request 1 has left before the failure
    assert not b.state and b.free == [0, 1, 2]

    def boom(i, t):
        raise KeyError("callback")

    b = Scripted(n_slots=2)
    with pytest.raises(KeyError):
        generate_ids(b, [[10], [20]], max_tokens=5, on_token=boom)
    assert not b.state and b.free == [0, 1]
    assert generate_ids(b, [[10], [20]], max_tokens=1) == [[11], [21]]               # and the backend is usable again


def test_streaming_callback_and_keys():
    seen = []
    b = Scripted(n_slots=2)
    generate_ids(b, [[10], [20]], max_tokens=2, on_token=lambda i, t: seen.append((i, t)))
    assert seen == [(0, 11), (1, 21), (0, 12), (1, 22)]
    assert stream_key(1, 0) != stream_key(1, 1) != stream_key(2, 1)
    assert -(1 << 63) <= stream_key(123, 4) < (1 << 63)


class ScriptedAhead(Scripted):
    """The same sequences behind a backend that launches steps without waiting: a launched step's tokens exist
    only when it is finished, a step launched after another feeds each sequence what that one sampled, at most two
    steps are in flight, and no step is begun or launched ahead for a slot that is known to be given back."""

    def __init__(self, *a, ahead_from=0, **kw):
        super().__init__(*a, **kw)
        self.in_flight = []
        self.serial = 0
        self.ahead_from = ahead_from          # begin_after answers None for the first steps (as uncaptured steps do)
        self.seq = {}                         # slot -> [first prompt token, steps launched]

    def open(self):
        s = super().open()
        self.seq[s] = None
        return s

    def _launch(self, slots, feeds, kind):
        assert len(self.in_flight) < 2, "more than two steps in flight"
        for s in slots:
            assert s in self.state, "a step was launched for a slot that is not held"
        self.serial += 1
        out = []
        for s, f in zip(slots, feeds):
            if self.seq[s] is None:
                self.seq[s] = [f[0], 0]
            elif f is not None:
                assert f == [self.seq[s][0] + self.seq[s][1]], "fed something else than the token sampled last"
            self.seq[s][1] += 1
            out.append(self.seq[s][0] + self.seq[s][1])
        h = {"slots": list(slots), "out": out}
        self.in_flight.append(h)
        self.log.append((kind, list(slots)))
        return h

    def begin(self, slots, feeds, keys, params):
        return self._launch(slots, feeds, "begin")

    def begin_after(self, pending):
        if self.serial < self.ahead_from:
            return None
        assert pending in self.in_flight, "launched after a step that was already finished"
        return self._launch(pending["slots"], [None] * len(pending["slots"]), "ahead")

    def finish(self, pending):
        assert self.in_flight and self.in_flight[0] is pending, "steps are finished in the order of their launch"
        self.in_flight.pop(0)
        return pending["out"]


def _ahead(**kw):
    return ScriptedAhead(**kw)


@pytest.mark.parametrize("ahead_from", [0, 3])
def test_steps_launched_ahead_give_the_tokens_of_steps_run_one_by_one(ahead_from):
    import random
    rng = random.Random(5)
    for trial in range(60):
        n = rng.randint(1, 7)
        prompts = [[rng.randint(1, 40) * 10] + [1] * rng.randint(0, 5) for _ in range(n)]
        kw = dict(max_tokens=rng.randint(0, 9), stop_token_ids=[rng.randint(1, 40) * 10 + rng.randint(1, 9) for _ in range(3)],
                  max_batch=rng.choice([None, 2, 3]), context_limit=rng.choice([None, 9, 12]))
        slots = rng.randint(1, 4)
        want_stats, got_stats = GenerationStats(), GenerationStats()
        want = generate_ids(Scripted(n_slots=slots), prompts, stats=want_stats, **kw)
        b = _ahead(n_slots=slots, ahead_from=ahead_from)
        got = generate_ids(b, prompts, stats=got_stats, **kw)
        assert got == want, (trial, prompts, kw)
        assert not b.state and not b.in_flight and sorted(b.free) == list(range(slots))
        assert got_stats.generated_tokens == want_stats.generated_tokens and got_stats.batches == want_stats.batches
        assert got_stats.prompt_tokens == want_stats.prompt_tokens


def test_a_stop_token_costs_one_row_of_the_step_that_ran_ahead():
    b = _ahead(n_slots=2)
    out = generate_ids(b, [[10], [20]], max_tokens=6, stop_token_ids=[13])
    assert out == [[11, 12], [21, 22, 23, 24, 25, 26]]
    kinds = [e for e in b.log if e[0] in ("begin", "ahead")]
    # prompts, two steps ahead (the second carries the sequence that its predecessor ends), one step begun anew
    # for the sequence that is left, then ahead again; the last step is not launched ahead: the count limit is known
    assert kinds[:4] == [("begin", [0, 1]), ("ahead", [0, 1]), ("ahead", [0, 1]), ("ahead", [0, 1])]
    assert kinds[4] == ("begin", [1]) and all(k == ("ahead", [1]) for k in kinds[5:])
    i_close = b.log.index(("close", 0))
    assert b.log[i_close - 1][0] == "ahead"       # the slot was given back while the step that ran ahead was in flight


def test_a_failure_with_a_step_in_flight_gives_every_slot_back():
    b = _ahead(n_slots=3)

    def boom(i, tok):
        if tok == 12:
            raise RuntimeError("callback")
    with pytest.raises(RuntimeError):
        generate_ids(b, [[10], [20], [30]], max_tokens=5, on_token=boom)
    assert not b.state and sorted(b.free) == [0, 1, 2]


def test_decode_split_rule_is_fixed_within_a_graph_class():
    """A captured decode graph is keyed by the class of the longest sequence: within a class the number of page
    splits must not change, for any batch size, and it never asks for more CTAs than the rule allows."""
    from gguf_rs_cli_b200 import kernels
    sms = 148
    for heads, kv in ((32, 8), (40, 40), (6, 3), (32, 1)):
        for T in (1, 2, 3, 8, 16, 64, 200):
            seen = {}
            for max_kv in list(range(1, 3000, 7)) + list(range(3000, 140000, 997)):
                cls = kernels.decode_split_class(max_kv)
                s = kernels.decode_splits(T, heads, kv, max_kv, sms, True)
                assert seen.setdefault(cls, s) == s, (heads, kv, T, max_kv)
                pages = (max_kv + 63) // 64
                group = heads // kv
                ctas = T * kv * ((group + 15) // 16)
                assert 1 <= s <= max(1, pages) and (s == 1 or s * ctas <= 2 * sms)
    assert kernels.decode_splits(1, 32, 8, 2048, sms, True) == 8 and kernels.decode_splits(8, 32, 8, 520, sms, True) == 1
    # eight sequences split in two from about 1,500 positions on, sixteen never: one CTA per SM is kept
    assert [kernels.decode_splits(8, 32, 8, n, sms, True) for n in (1024, 1600, 2048, 8000)] == [1, 2, 2, 2]
    assert kernels.decode_splits(16, 32, 8, 4096, sms, True) == 1 and kernels.decode_splits(4, 32, 8, 4096, sms, True) == 4

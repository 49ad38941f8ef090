"""Generation through the Python entry point against the plain implementation."""
import pytest
import torch

from tests import plain_llama as P
from tests.gpu_util import assert_close, llm, new_engine, plain_logits, plain_weights, tokens_of
from tests.tiny import config

pytestmark = pytest.mark.gpu


def plain_generate(name, prompts, max_tokens, **kw):
    cfg, w = config(name), plain_weights(name)
    return [P.generate(cfg, w, p, max_tokens, index=i, **kw) for i, p in enumerate(prompts)]


def test_greedy_generation_float32_equals_plain():
    from gguf_rs_cli_b200.api import generate
    prompts = [tokens_of("A", n, 50 + n) for n in (5, 9, 13)]
    want = plain_generate("A", prompts, 8)
    got = generate(llm("A", "float32"), prompts, max_tokens=8, temperature=0.0, stop_token_ids=[])
    assert got == want


def test_seeded_temperature_generation_equals_plain():
    from gguf_rs_cli_b200.api import generate
    prompts = [tokens_of("B", n, 60 + n) for n in (1, 7, 20, 33)]
    want = plain_generate("B", prompts, 12, temperature=0.8, seed=1234)
    got = generate(llm("B", "float32"), prompts, max_tokens=12, temperature=0.8, seed=1234, stop_token_ids=[])
    assert got == want
    other = generate(llm("B", "float32"), prompts, max_tokens=12, temperature=0.8, seed=99, stop_token_ids=[])
    assert other != got
    # a request's draws do not depend on its batch: alone it gives the same tokens (its index is its stream)
    alone = generate(llm("B", "float32"), prompts[:1], max_tokens=12, temperature=0.8, seed=1234, stop_token_ids=[])
    assert alone[0] == got[0]


def test_reference_defaults_top_k_top_p_penalty():
    from gguf_rs_cli_b200.api import generate
    prompts = [tokens_of("A", n, 70 + n) for n in (4, 11)]
    kw = dict(temperature=0.7, top_k=40, top_p=0.9, rep_penalty=1.1, seed=42)
    want = plain_generate("A", prompts, 10, **kw)
    got = generate(llm("A", "float32"), prompts, max_tokens=10, stop_token_ids=[], **kw)
    assert got == want


def test_bfloat16_greedy_follows_plain_until_a_near_tie():
    from gguf_rs_cli_b200.api import generate
    cfg, w = config("C"), plain_weights("C")
    prompts = [tokens_of("C", n, 80 + n) for n in (3, 40, 70)]
    got = generate(llm("C", "bfloat16"), prompts, max_tokens=12, temperature=0.0, stop_token_ids=[])
    for p, g in zip(prompts, got):
        seq = list(p)
        for tok in g:
            logits = P.forward(cfg, w, seq)[-1]
            best = float(logits.max())
            # the engine's choice is the plain argmax, or within bfloat16 noise of it
            assert float(logits[tok]) >= best - 2e-2 * float(logits.abs().max()), f"token {tok} at length {len(seq)}"
            seq.append(tok)


def test_stop_tokens_batches_and_slot_reuse():
    from gguf_rs_cli_b200.api import generate
    from gguf_rs_cli_b200.engine.generate import GenerationStats
    model = llm("A", "float32")
    prompts = [tokens_of("A", 3 + (i * 5) % 17, 90 + i) for i in range(7)]
    free = plain_generate("A", prompts, 10)
    stop = free[2][4]
    want = plain_generate("A", prompts, 10, stop=[stop])
    stats = GenerationStats()
    got = generate(model, prompts, max_tokens=10, stop_token_ids=[stop], max_batch=3, stats=stats)
    assert got == want and stats.batches == 3
    assert len(got[2]) <= 4 and stop not in got[2]
    assert model._engine.cache.slots.held_count == 0
    model._engine.cache.check()
    # eos from config.json is the default stop set
    assert model.spec.stop_token_ids == [2]


def test_context_limit_and_long_decoding():
    from gguf_rs_cli_b200.api import generate
    prompts = [tokens_of("A", 5, 7)]
    want = plain_generate("A", prompts, 500, max_len=40)
    got = generate(llm("A", "float32"), prompts, max_tokens=500, ctx_len=40, stop_token_ids=[])
    assert got == want and len(got[0]) == 40 - 1 - 5
    # long decoding across several pages: logits of each decoded position against the plain ones
    for dtype in ("float32", "bfloat16"):
        eng = new_engine("B", dtype, n_tokens=512, n_slots=2)
        from gguf_rs_cli_b200.engine.step import Entry
        n = 230
        toks, ref = tokens_of("B", n, 3), plain_logits("B", n, 3)
        s = eng.open()
        eng.step([Entry(s, toks[:2], [])])
        for i in range(2, n):
            got_l = eng.step([Entry(s, [toks[i]], [0])])
            if i % 7 == 0 or i > n - 5 or i in (63, 64, 65, 127, 128, 129):
                assert_close(got_l[0], ref[i], dtype, f"decoded position {i}")
        eng.close(s)


def test_graph_and_eager_decode_agree():
    """The captured decode step gives the tokens of the eager one, also when the batch
    shrinks inside a padded bucket."""
    from gguf_rs_cli_b200.engine.backend import EngineBackend
    from gguf_rs_cli_b200.engine.generate import generate_ids
    from gguf_rs_cli_b200.sampling import SamplingParams
    prompts = [tokens_of("C", n, 200 + n) for n in (3, 70, 9, 20, 64)]
    outs = []
    for graphs in (False, True):
        eng = new_engine("C", "bfloat16", n_tokens=64 * 16, n_slots=8)
        backend = EngineBackend(eng, use_graphs=graphs)
        stops = []
        outs.append(generate_ids(backend, prompts, 9, SamplingParams(temperature=0.9, seed=5), stops))
        free = outs[-1]
        stop = free[1][3]
        outs.append(generate_ids(backend, prompts, 9, SamplingParams(temperature=0.9, seed=5), [stop]))
        assert eng.cache.slots.held_count == 0
    assert outs[0] == outs[2] and outs[1] == outs[3]


@pytest.mark.parametrize("name", ["C", "D"])
def test_bfloat16_sampling_options_through_captured_graphs(name):
    """top_k, top_p and the repetition penalty (the reference's defaults) in bfloat16: the captured decode
    step (sampling inside the graph, its recent-token ring in the per-sequence state) gives the tokens of steps
    launched one by one, also for a second batch in used slots; and every token chosen is one that the plain
    sampler could choose from the plain logits (inside its top_k by the margin of bfloat16)."""
    from gguf_rs_cli_b200.engine.backend import EngineBackend
    from gguf_rs_cli_b200.engine.generate import generate_ids
    from gguf_rs_cli_b200.sampling import SamplingParams
    cfg, w = config(name), plain_weights(name)
    prompts = [tokens_of(name, n, 400 + n) for n in (5, 66, 31)]
    params = SamplingParams(temperature=0.7, top_k=40, top_p=0.9, rep_penalty=1.1, seed=11)
    outs = []
    for graphs in (False, True):
        eng = new_engine(name, "bfloat16", n_tokens=64 * 8, n_slots=4)
        backend = EngineBackend(eng, use_graphs=graphs)
        outs.append([generate_ids(backend, prompts, 14, params, []) for _ in range(2)])
        assert outs[-1][0] == outs[-1][1], "the second batch reuses slots whose ring of recent tokens must start empty"
    assert outs[0] == outs[1]
    for p, g in zip(prompts, outs[1][0]):
        seq, recent = list(p), []
        for tok in g:
            logits = P.apply_rep_penalty(P.forward(cfg, w, seq)[-1], recent, 1.1)
            kth = float(torch.topk(logits, 40).values[-1])
            assert float(logits[tok]) >= kth - 2e-2 * float(logits.abs().max()), f"token {tok} at length {len(seq)} is outside top_k"
            seq.append(tok)
            recent = (recent + [tok])[-64:]


@pytest.mark.parametrize("name", ["B", "C"])
def test_decode_steps_updated_in_place_cross_pages(name):
    """While a batch goes on token by token, the captured step's index arrays are only
    updated; sequences that enter a new page (positions 64, 128) and one that ends early
    must give the tokens of the step that is laid out anew every time, and of the plain code."""
    from gguf_rs_cli_b200.engine.backend import EngineBackend
    from gguf_rs_cli_b200.engine.generate import generate_ids
    from gguf_rs_cli_b200.sampling import SamplingParams
    prompts = [tokens_of(name, n, 300 + n) for n in (60, 3, 125, 62, 64)]
    want = plain_generate(name, prompts, 10)
    params = SamplingParams(temperature=0.0)
    for graphs in (False, True):
        eng = new_engine(name, "float32", n_tokens=64 * 24, n_slots=8)
        backend = EngineBackend(eng, use_graphs=graphs)
        for _ in range(2):                                   # the second pass replays captured graphs on used slots
            got = generate_ids(backend, prompts, 10, params, [])
            assert got == want
            eng.cache.check()
        stop = want[1][4]
        got = generate_ids(backend, prompts, 10, params, [stop])
        for g, w in zip(got, want):
            assert g == (w[:w.index(stop)] if stop in w else w)        # the stop token itself is not given out
        assert eng.cache.slots.held_count == 0
        # captured steps are launched before the tokens of the step in front of them are read; others are not
        assert (backend.steps_ahead >= 20) if graphs else backend.steps_ahead == 0


def test_decode_past_a_thousand_positions_splits_pages_and_changes_graphs():
    """Two sequences of the wide tiny model decode across position 960, where the decode attention goes from one
    split of a sequence's pages to four (another captured graph from there on): the captured steps give the
    tokens of the eager ones, and the logits on both sides of the change are the plain implementation's."""
    from gguf_rs_cli_b200.engine.backend import EngineBackend
    from gguf_rs_cli_b200.engine.generate import generate_ids
    from gguf_rs_cli_b200.engine.step import Entry
    from gguf_rs_cli_b200.sampling import SamplingParams
    assert config("C")["max_position_embeddings"] >= 1024
    prompts = [tokens_of("C", n, 500 + n) for n in (945, 930)]
    outs = []
    for graphs in (False, True):
        eng = new_engine("C", "bfloat16", n_tokens=64 * 34, n_slots=2)
        outs.append(generate_ids(EngineBackend(eng, use_graphs=graphs), prompts, 40, SamplingParams(temperature=0.0), []))
        assert eng.cache.slots.held_count == 0
    assert outs[0] == outs[1]
    # logits of single-token steps at positions 940..985 of one long sequence against the plain ones
    n = 986
    toks, ref = tokens_of("C", n, 77), plain_logits("C", n, 77)
    eng = new_engine("C", "bfloat16", n_tokens=64 * 34, n_slots=2)
    a, b = eng.open(), eng.open()
    eng.step([Entry(a, toks[:940], []), Entry(b, toks[:100], [])])
    for i in range(940, n):
        got = eng.step([Entry(a, [toks[i]], [0]), Entry(b, [toks[100 + i - 940]], [])])
        assert_close(got[0], ref[i], "bfloat16", f"decoded position {i}")

"""The engine against the plain implementation, in 32-bit and in bfloat16: requests
alone and whole, the last 32 tokens one by one, batches of unequal lengths whose
shorter requests end earlier, one batch after another so that slots are used again."""
import pytest
import torch

from tests.gpu_util import assert_close, new_engine, plain_logits, tokens_of

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
NAMES = ["A", "B", "C", "D"]


def entry(slot, tokens, want):
    from gguf_rs_cli_b200.engine.step import Entry
    return Entry(slot, tokens, want)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES + ["E"])
def test_whole_request_alone(name, dtype):
    eng = new_engine(name, dtype)
    for n, seed in [(1, 1), (5, 2), (33, 3), (100, 4)]:
        toks = tokens_of(name, n, seed)
        s = eng.open()
        got = eng.step([entry(s, toks, range(n))])
        eng.close(s)
        assert_close(got, plain_logits(name, n, seed), dtype, f"{name} whole n={n}")
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES + ["E"])
def test_last_32_one_by_one(name, dtype):
    eng = new_engine(name, dtype)
    n, seed = 90, 7
    toks, want = tokens_of(name, n, seed), plain_logits(name, n, seed)
    s = eng.open()
    head = eng.step([entry(s, toks[:n - 32], range(n - 32))])
    assert_close(head, want[:n - 32], dtype, "prefix")
    for i in range(n - 32, n):
        got = eng.step([entry(s, [toks[i]], [0])])
        assert_close(got[0], want[i], dtype, f"{name} decoded position {i}")
    eng.close(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_one_after_another(name, dtype):
    eng = new_engine(name, dtype, n_tokens=64 * 8, n_slots=4)
    lens_per_batch = [[5, 9, 13, 70], [1, 7, 20, 33], [64, 65, 2]]
    decode = 6
    seed = 100
    for lens in lens_per_batch:
        reqs = []
        for n in lens:
            seed += 1
            total = n + decode
            reqs.append(dict(toks=tokens_of(name, total, seed), want=plain_logits(name, total, seed), n=n,
                             keep=decode - (seed % 3), slot=eng.open(), fed=0))
        got = eng.step([entry(r["slot"], r["toks"][:r["n"]], [r["n"] - 1]) for r in reqs])
        for i, r in enumerate(reqs):
            assert_close(got[i], r["want"][r["n"] - 1], dtype, f"{name} prompt of {r['n']} in batch {lens}")
            r["fed"] = r["n"]
        live = list(reqs)
        for step in range(decode):
            live = [r for r in live if r["fed"] < r["n"] + r["keep"]]          # shorter ones end earlier
            for r in reqs:
                if r not in live and r["slot"] is not None:
                    eng.close(r["slot"])
                    r["slot"] = None
            if not live:
                break
            got = eng.step([entry(r["slot"], [r["toks"][r["fed"]]], [0]) for r in live])
            for i, r in enumerate(live):
                assert_close(got[i], r["want"][r["fed"]], dtype, f"{name} step {step} of prompt {r['n']}")
                r["fed"] += 1
        for r in reqs:
            if r["slot"] is not None:
                eng.close(r["slot"])
        eng.cache.check()
    assert eng.cache.slots.held_count == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_continuation_in_pieces_and_nothing_wanted(dtype):
    name = "B"
    eng = new_engine(name, dtype)
    n, seed = 75, 11
    toks, want = tokens_of(name, n, seed), plain_logits(name, n, seed)
    s = eng.open()
    assert eng.step([entry(s, toks[:10], [])]) is None
    got = eng.step([entry(s, toks[10:63], [0, 52])])
    assert_close(got, want[[10, 62]], dtype, "second piece")
    got = eng.step([entry(s, toks[63:], range(n - 63))])
    assert_close(got, want[63:], dtype, "third piece across a page boundary")
    eng.close(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["C", "D"])
def test_a_new_prompt_joins_sequences_that_are_decoding(name, dtype):
    """One step that mixes two sequences going on by one token (at positions past a page boundary) with a
    prompt that starts: the tiled prompt kernels (tensor cores at head sizes 64 and 128) then see rows of one
    query at start > 0 beside a whole prompt.  Every entry's logits are checked, before, in and after the
    mixed step."""
    eng = new_engine(name, dtype, n_tokens=64 * 12, n_slots=4)
    lens = {"a": 150, "b": 75, "c": 49}
    toks = {r: tokens_of(name, n, 40 + n) for r, n in lens.items()}
    want = {r: plain_logits(name, n, 40 + n) for r, n in lens.items()}
    slot = {r: eng.open() for r in "ab"}
    fed = {"a": 140, "b": 66}
    got = eng.step([entry(slot[r], toks[r][:fed[r]], [fed[r] - 1]) for r in "ab"])
    for i, r in enumerate("ab"):
        assert_close(got[i], want[r][fed[r] - 1], dtype, f"{name} prompt {r}")
    for _ in range(2):
        got = eng.step([entry(slot[r], [toks[r][fed[r]]], [0]) for r in "ab"])
        for i, r in enumerate("ab"):
            assert_close(got[i], want[r][fed[r]], dtype, f"{name} {r} at {fed[r]}")
            fed[r] += 1
    slot["c"] = eng.open()
    got = eng.step([entry(slot["a"], [toks["a"][fed["a"]]], [0]), entry(slot["c"], toks["c"][:45], range(45)),
                    entry(slot["b"], [toks["b"][fed["b"]]], [0])])
    assert_close(got[0], want["a"][fed["a"]], dtype, f"{name} a in the mixed step")
    assert_close(got[1:46], want["c"][:45], dtype, f"{name} the joining prompt")
    assert_close(got[46], want["b"][fed["b"]], dtype, f"{name} b in the mixed step")
    fed["a"] += 1
    fed["b"] += 1
    fed["c"] = 45
    for _ in range(4):
        got = eng.step([entry(slot[r], [toks[r][fed[r]]], [0]) for r in "abc"])
        for i, r in enumerate("abc"):
            assert_close(got[i], want[r][fed[r]], dtype, f"{name} {r} at {fed[r]} after the mixed step")
            fed[r] += 1
    for r in "abc":
        eng.close(slot[r])
    eng.cache.check()


@pytest.mark.parametrize("name", NAMES)
def test_float32_logits_do_not_depend_on_the_cut_to_the_bit(name):
    """In 32-bit mode every product is one thread's sum in ascending k and attention runs its blocks in a fixed
    order, so whole prompts, tokens one by one and unequal batches give the same bits."""
    eng = new_engine(name, "float32", n_tokens=64 * 10, n_slots=4)
    n = 80
    toks = tokens_of(name, n, 5)
    other = tokens_of(name, 60, 6)
    s = eng.open()
    whole = eng.step([entry(s, toks, range(n))]).clone()
    eng.close(s)
    # the last 32 one by one, in a slot used before, beside another sequence
    o, s = eng.open(), eng.open()
    head = eng.step([entry(o, other[:20], [19]), entry(s, toks[:n - 32], range(n - 32))])
    assert torch.equal(head[1:], whole[:n - 32]), "a prompt beside another one"
    for i in range(n - 32, n):
        got = eng.step([entry(s, [toks[i]], [0]), entry(o, [other[20 + i - (n - 32)]], [])] if i % 2 else [entry(s, [toks[i]], [0])])
        assert torch.equal(got[0], whole[i]), f"position {i} decoded"
    eng.close(s)
    eng.close(o)
    # in three pieces cut inside a page
    s = eng.open()
    a = eng.step([entry(s, toks[:7], range(7))]).clone()
    b = eng.step([entry(s, toks[7:70], range(63))]).clone()
    c = eng.step([entry(s, toks[70:], range(10))]).clone()
    assert torch.equal(torch.cat([a, b, c]), whole)
    eng.close(s)


def test_captured_graphs_survive_a_later_large_step():
    """Decode graphs captured early keep the addresses of the scratch memory that split products and split
    attention share.  A later step with larger needs (a prompt of a few hundred tokens at the benchmark's layer
    width) must not move that memory under them: the tokens decoded afterwards through the old graphs equal
    those of steps that are launched one by one."""
    from gguf_rs_cli_b200.api import from_random
    from gguf_rs_cli_b200.engine.backend import EngineBackend
    from gguf_rs_cli_b200.engine.generate import generate_ids
    from gguf_rs_cli_b200.engine.step import Engine
    from gguf_rs_cli_b200.sampling import SamplingParams
    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 1, "hidden_size": 4096,
           "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336,
           "vocab_size": 4096, "rope_theta": 500000.0, "rms_norm_eps": 1e-5, "max_position_embeddings": 1024,
           "tie_word_embeddings": True, "hidden_act": "silu"}
    model = from_random(cfg, seed=3, dtype="bfloat16", device="cuda:0").model
    g = torch.Generator().manual_seed(2)
    short = [torch.randint(0, 4096, (10,), generator=g).tolist()]
    long = [torch.randint(0, 4096, (n,), generator=g).tolist() for n in (200, 333)]
    params = SamplingParams(temperature=0.0)
    outs = []
    for graphs in (True, False):
        backend = EngineBackend(Engine(model, n_tokens=64 * 16, n_slots=4, max_len=1024), use_graphs=graphs)
        first = generate_ids(backend, short, 6, params, [])          # captures the graph of one sequence
        generate_ids(backend, long, 3, params, [])                   # a step of 533 tokens, then graphs of two sequences
        again = generate_ids(backend, short, 6, params, [])          # replays the first graph
        assert first == again
        outs.append((first, again))
    assert outs[0] == outs[1]
    del model
    torch.cuda.empty_cache()


def test_step_errors_launch_nothing():
    from gguf_rs_cli_b200.cache import CacheError, CacheFull
    from gguf_rs_cli_b200.engine.step import StepError
    eng = new_engine("A", "float32", n_tokens=128, n_slots=2)
    s = eng.open()
    with pytest.raises(StepError, match="token id 256"):
        eng.step([entry(s, [1, 256], [0])])
    with pytest.raises(StepError, match="at least one token"):
        eng.step([entry(s, [], [])])
    with pytest.raises(StepError, match="wanted place"):
        eng.step([entry(s, [1, 2], [2])])
    with pytest.raises(CacheError, match="not open"):
        eng.step([entry(1, [1], [0])])
    with pytest.raises(CacheFull):
        eng.step([entry(s, [1] * 129, [0])])
    assert eng.cache.length(s) == 0
    eng.close(s)
    eng.cache.check()


@pytest.mark.parametrize("lens", [(700, 300, 64), tuple(20 + 2 * i for i in range(40))], ids=["3 long", "40 short"])
def test_bfloat16_path_against_the_32_bit_path_at_the_benchmark_layer_sizes(lens):
    """Two layers of the Llama-3.1-8B layer shape (head size 128, 32 heads in 8 groups, widths 4096 / 14336;
    a smaller vocabulary) with random weights: prompts of unequal lengths in one step (the tensor-core
    attention and the two-SM product run here, which the tiny models do not reach), then single tokens; the
    bfloat16 logits against the true 32-bit path's.  With 40 sequences the decode steps take what a large batch
    takes: tiles of 64 tokens that several CTAs share and finish a share each, and the attention kernel's CTAs of
    two warps."""
    from gguf_rs_cli_b200.api import from_random
    from gguf_rs_cli_b200.engine.step import Engine, Entry
    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 2, "hidden_size": 4096,
           "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336,
           "vocab_size": 8192, "rope_theta": 500000.0,
           "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                            "original_max_position_embeddings": 8192},
           "rms_norm_eps": 1e-5, "max_position_embeddings": 2048, "tie_word_embeddings": False, "hidden_act": "silu"}
    g = torch.Generator().manual_seed(1)
    toks = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]
    res = {}
    for dtype in ("float32", "bfloat16"):
        model = from_random(cfg, seed=0, dtype=dtype, device="cuda:0").model
        eng = Engine(model, n_tokens=64 * max(24, 2 * len(lens)), n_slots=len(lens) + 1, max_len=2048)
        slots = [eng.open() for _ in toks]
        out = [eng.step([Entry(s, t[:-8], [len(t) - 9, 0, len(t) // 2]) for s, t in zip(slots, toks)])]
        for i in range(8, 0, -1):
            out.append(eng.step([Entry(s, [t[-i]], [0]) for s, t in zip(slots, toks)]))
        res[dtype] = torch.cat(out).float().cpu()
        del model, eng
        torch.cuda.empty_cache()
    assert_close(res["bfloat16"], res["float32"], "bfloat16", "8B layer shape")

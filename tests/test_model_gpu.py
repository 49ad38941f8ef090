"""The engine against the plain implementation, in 32-bit and in bfloat16: requests
alone and whole, the last 32 tokens one by one, batches of unequal lengths whose
shorter requests end earlier, one batch after another so that slots are used again."""
import pytest
import torch

from tests.gpu_util import assert_close, new_engine, plain_logits, tokens_of

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
NAMES = ["A", "B", "C"]


def entry(slot, tokens, want):
    from gguf_rs_cli_b200.engine.step import Entry
    return Entry(slot, tokens, want)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
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
@pytest.mark.parametrize("name", NAMES)
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


def test_bfloat16_path_against_the_32_bit_path_at_the_benchmark_layer_sizes():
    """Two layers of the Llama-3.1-8B layer shape (head size 128, 32 heads in 8 groups, widths 4096 / 14336;
    a smaller vocabulary) with random weights: prompts of unequal lengths in one step (the tensor-core
    attention and the two-SM product run here, which the tiny models do not reach), then single tokens; the
    bfloat16 logits against the true 32-bit path's."""
    from gguf_rs_cli_b200.api import from_random
    from gguf_rs_cli_b200.engine.step import Engine, Entry
    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 2, "hidden_size": 4096,
           "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336,
           "vocab_size": 8192, "rope_theta": 500000.0,
           "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                            "original_max_position_embeddings": 8192},
           "rms_norm_eps": 1e-5, "max_position_embeddings": 2048, "tie_word_embeddings": False, "hidden_act": "silu"}
    g = torch.Generator().manual_seed(1)
    toks = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in (700, 300, 64)]
    res = {}
    for dtype in ("float32", "bfloat16"):
        model = from_random(cfg, seed=0, dtype=dtype, device="cuda:0").model
        eng = Engine(model, n_tokens=64 * 24, n_slots=4, max_len=2048)
        slots = [eng.open() for _ in toks]
        out = [eng.step([Entry(s, t[:-8], [len(t) - 9, 0, len(t) // 2]) for s, t in zip(slots, toks)])]
        for i in range(8, 0, -1):
            out.append(eng.step([Entry(s, [t[-i]], [0]) for s, t in zip(slots, toks)]))
        res[dtype] = torch.cat(out).float().cpu()
        del model, eng
        torch.cuda.empty_cache()
    assert_close(res["bfloat16"], res["float32"], "bfloat16", "8B layer shape")

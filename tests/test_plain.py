"""The plain implementation against itself: formulas that can be checked by hand."""
import math

import torch

from tests import plain_llama as P
from tests.tiny import config


def test_rmsnorm_by_hand():
    x = torch.tensor([[3.0, 4.0]])
    out = P.rmsnorm(x, torch.tensor([2.0, 0.5]), 0.0)
    rms = math.sqrt(12.5)
    assert torch.allclose(out, torch.tensor([[3 / rms * 2, 4 / rms * 0.5]]))


def test_rope_pairs_halves_and_keeps_position_zero():
    cfg = {"hidden_size": 8, "num_attention_heads": 1, "rope_theta": 10000.0}
    f = P.inv_freq_table(cfg)
    assert torch.allclose(f, torch.tensor([1.0, 10000 ** -0.25, 10000 ** -0.5, 10000 ** -0.75]))
    x = torch.arange(8.0).reshape(1, 1, 8)
    assert torch.equal(P.rope(x, torch.tensor([0]), f), x)
    y = P.rope(x, torch.tensor([1]), f)[0, 0]
    assert abs(float(y[0]) - (0 * math.cos(1) - 4 * math.sin(1))) < 1e-6
    assert abs(float(y[4]) - (0 * math.sin(1) + 4 * math.cos(1))) < 1e-6


def test_llama3_bands():
    cfg = config("B")
    plain = dict(cfg, rope_scaling=None)
    f0, f = P.inv_freq_table(plain, torch.float64), P.inv_freq_table(cfg, torch.float64)
    ratio = (f / f0)
    assert abs(float(ratio[0]) - 1.0) < 1e-6 and abs(float(ratio[-1]) - 1 / 8) < 1e-6     # kept / divided
    assert any(0.13 < float(r) < 0.99 for r in ratio)                  # and a blended band between


def test_attention_is_causal_and_grouped():
    torch.manual_seed(0)
    q, k, v = torch.randn(5, 4, 8), torch.randn(5, 2, 8), torch.randn(5, 2, 8)
    a = P.attention(q, k, v)
    k2, v2 = k.clone(), v.clone()
    k2[3:], v2[3:] = 9.0, 9.0                      # the future does not reach positions 0..2
    assert torch.equal(P.attention(q, k2, v2)[:3], a[:3])
    assert torch.allclose(a[0].reshape(4, 8), v[0][[0, 0, 1, 1]])       # one key: its value; heads 0,1 -> kv 0
    w = P.attention(q, k, v, window=2)
    assert torch.allclose(w[1], a[1]) and not torch.allclose(w[4], a[4])


def test_forward_prefix_property_and_tied_head():
    cfg = config("B")
    w = P.random_weights(cfg, 1)
    toks = [3, 9, 200, 17, 5, 300]
    full = P.forward(cfg, w, toks)
    assert full.shape == (6, 384)
    assert torch.allclose(P.forward(cfg, w, toks[:4]), full[:4], atol=1e-6)
    f64 = P.forward(cfg, w, toks, torch.float64)
    assert float((full.double() - f64).abs().max()) < 1e-5


def test_sampler_rules():
    logits = torch.tensor([1.0, 3.0, 2.0, 3.0, -1.0])
    assert P.greedy(logits) == 1
    pen = P.apply_rep_penalty(logits, [1, 4, 4], 2.0)
    assert pen.tolist() == [1.0, 1.5, 2.0, 3.0, -4.0]
    assert P.sample(logits, 0.0, 0, 1.0, 1.0, [], 0.99) == 1
    assert P.sample(logits, 1.0, 1, 1.0, 1.0, [], 0.99) == 1                 # top_k 1: the first maximum
    assert P.sample(logits, 1.0, 2, 1.0, 1.0, [], 0.99) == 3                 # top_k 2: both maxima, walk in index order
    assert P.sample(logits, 1.0, 0, 0.3, 1.0, [], 0.99) == 1                 # top_p below the first mass
    counts = [0] * 5
    for n in range(2000):
        counts[P.sample(logits, 1.0, 0, 1.0, 1.0, [], P.uniform(7, n))] += 1
    p = torch.softmax(logits, 0)
    assert all(abs(c / 2000 - float(pi)) < 0.04 for c, pi in zip(counts, p))
    us = [P.uniform(P.mix_seed(42, 0), n) for n in range(1000)]
    assert 0 <= min(us) and max(us) < 1 and 0.45 < sum(us) / 1000 < 0.55


def test_generate_stops():
    cfg = config("A")
    w = P.random_weights(cfg, 3)
    out = P.generate(cfg, w, [5, 6, 7], max_tokens=4)
    assert len(out) == 4
    assert P.generate(cfg, w, [5, 6, 7], max_tokens=4, stop=[out[2]]) == out[:2]
    assert P.generate(cfg, w, [5, 6, 7], max_tokens=40, max_len=6) == out[:2]

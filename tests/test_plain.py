"""The plain implementation against itself: formulas that can be checked by hand."""
import math

import pytest
import torch

from tests import plain_llama as P
from tests.tiny import config, qk_std


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


def test_softmax_silu_and_linear_by_hand():
    """src/math/ops.rs:5-11 and src/tensor/dequant.rs:315-317 on numbers small enough to do by hand."""
    s = P.softmax(torch.tensor([[0.0, math.log(3.0)]]))
    assert torch.allclose(s, torch.tensor([[0.25, 0.75]]))
    big = P.softmax(torch.tensor([[1000.0, 1000.0]]))              # the maximum is subtracted first
    assert torch.allclose(big, torch.tensor([[0.5, 0.5]]))
    assert abs(float(P.silu(torch.tensor(0.0)))) == 0.0
    assert abs(float(P.silu(torch.tensor(2.0))) - 2.0 / (1.0 + math.exp(-2.0))) < 1e-7
    w = torch.tensor([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]])         # [out, in]: y[i] = sum_j w[i, j] x[j]
    y = P.linear(torch.tensor([[1.0, -1.0]]), w, torch.tensor([0.5, 0.0, 0.0]))
    assert y.tolist() == [[-0.5, -1.0, -1.0]]
    ff = P.feed_forward(torch.tensor([[1.0, 0.0]]), torch.tensor([[2.0, 0.0]]), torch.tensor([[3.0, 0.0]]), torch.tensor([[1.0], [2.0]]))
    a = 2.0 / (1.0 + math.exp(-2.0)) * 3.0                         # silu(gate) * up, then down
    assert torch.allclose(ff, torch.tensor([[a, 2 * a]]))


def test_rmsnorm_has_eps_inside_the_root_and_rope_keeps_lengths():
    x = torch.zeros(1, 4)
    assert torch.equal(P.rmsnorm(x, torch.ones(4), 1e-5), x)        # 0 / sqrt(0 + eps)
    y = P.rmsnorm(torch.full((1, 4), 1e-3), torch.ones(4), 1e-6)    # mean square = eps: x / sqrt(2 eps)
    assert torch.allclose(y, torch.full((1, 4), 1e-3 / math.sqrt(2e-6)))
    f = P.inv_freq_table({"hidden_size": 16, "num_attention_heads": 2, "rope_theta": 100.0})
    q = torch.randn(3, 2, 8, generator=torch.Generator().manual_seed(0))
    r = P.rope(q, torch.tensor([0, 5, 77]), f)
    assert torch.allclose(r.norm(dim=-1), q.norm(dim=-1), atol=1e-5)
    # relative position only: <rope(q, m), rope(k, n)> depends on m - n
    k = torch.randn(1, 2, 8, generator=torch.Generator().manual_seed(1))
    d1 = (P.rope(q[:1], torch.tensor([9]), f) * P.rope(k, torch.tensor([4]), f)).sum()
    d2 = (P.rope(q[:1], torch.tensor([25]), f) * P.rope(k, torch.tensor([20]), f)).sum()
    assert abs(float(d1 - d2)) < 1e-4


def test_sampler_order_of_steps():
    """src/sampler.rs:35-79: penalty first, then temperature, then top_k on the scaled logits, softmax over
    the survivors, top_p on the descending order, renormalise, walk."""
    logits = torch.tensor([2.0, 1.0, 0.0, -1.0])
    # penalty before greedy: token 0 is halved and no longer the maximum
    assert P.sample(torch.tensor([2.0, 1.5, 0.0]), 0.0, 0, 1.0, 2.0, [0], 0.0) == 1
    # top_k 2 keeps tokens 0 and 1 with p = e/(1+e), 1/(1+e); u just above the first mass picks token 1
    p0 = math.e / (1 + math.e)
    assert P.sample(logits, 1.0, 2, 1.0, 1.0, [], p0 - 1e-3) == 0 and P.sample(logits, 1.0, 2, 1.0, 1.0, [], p0 + 1e-3) == 1
    # temperature divides before the softmax: at T = 0.5 the two survivors weigh e^2 : 1
    p0 = math.exp(2) / (1 + math.exp(2))
    assert P.sample(logits, 0.5, 2, 1.0, 1.0, [], p0 - 1e-3) == 0 and P.sample(logits, 0.5, 2, 1.0, 1.0, [], p0 + 1e-3) == 1
    # top_p cuts the smallest prefix whose mass reaches it (here 0.644 + 0.237 >= 0.8) and renormalises
    full = torch.softmax(logits, 0)
    cut = float(full[0] / (full[0] + full[1]))
    assert P.sample(logits, 1.0, 0, 0.8, 1.0, [], cut + 1e-3) == 1 and P.sample(logits, 1.0, 0, 0.8, 1.0, [], 0.999) == 1
    # a uniform at the very top returns the last survivor
    assert P.sample(logits, 1.0, 0, 1.0, 1.0, [], 1.0) == 3


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_the_test_weights_show_a_wrong_rotation_scaling_or_grouping(name, monkeypatch):
    """What the engine is compared against must move when the model is wrong.  With the weights the GPU tests
    use (q and k scaled so that attention is peaked), leaving the rotation out, dropping the frequency
    scaling, or reading the wrong KV head each move the logits by at least five times the bfloat16
    tolerance of those tests (2e-2 of the largest logit)."""
    cfg = config(name)
    w = P.random_weights(cfg, 0, norm_noise=0.1, qk_std=qk_std(cfg))
    w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, cfg["vocab_size"], (90,), generator=g).tolist()
    base = P.forward(cfg, w, toks)
    ref = float(base.abs().max())
    need = 5 * 2e-2

    def moved(other):
        return float((other - base).abs().max()) / ref

    with monkeypatch.context() as m:
        m.setattr(P, "rope", lambda x, positions, inv_freq: x)
        assert moved(P.forward(cfg, w, toks)) >= need, "no rotation"
    if cfg.get("rope_scaling"):
        assert moved(P.forward(dict(cfg, rope_scaling=None), w, toks)) >= need, "no frequency scaling"
    if P.kv_heads_of(cfg) > 1:
        real = P.attention

        def wrong_group(q, k, v, window=None):
            nh, nkv = q.shape[1], k.shape[1]
            order = [h % nkv for h in range(nh)]                 # head h reads KV head h % nkv instead of h // (nh/nkv)
            return real(q, k[:, order, :], v[:, order, :], window)

        with monkeypatch.context() as m:
            m.setattr(P, "attention", wrong_group)
            assert moved(P.forward(cfg, w, toks)) >= need, "wrong head group"
    # and the plain N(0, 0.02) weights would not have shown the rotation (which is why they are not used)
    flat = {k: v.to(torch.bfloat16).float() for k, v in P.random_weights(cfg, 0, norm_noise=0.1).items()}
    with monkeypatch.context() as m:
        flat_base = P.forward(cfg, flat, toks)
        m.setattr(P, "rope", lambda x, positions, inv_freq: x)
        assert float((P.forward(cfg, flat, toks) - flat_base).abs().max()) / float(flat_base.abs().max()) < need

"""Each part of a layer alone against the plain implementation, and the generality of
the composition: a toy mixer with state of its own (defined here, registered from
here), windowed and cache-sharing layers, a layer that runs twice; a toy feed-forward
that routes tokens to experts and a position encoding of its own in a second toy
architecture."""
import math
from dataclasses import dataclass

import pytest
import torch

from tests import plain_llama as P
from tests.gpu_util import TOL, assert_close, llm, new_engine, plain_weights, tokens_of
from tests.tiny import config

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = ["float32", "bfloat16"]


def tdtype(name):
    return {"float32": torch.float32, "bfloat16": torch.bfloat16}[name]


def plan_for(eng, lens, starts=None):
    """Opens one sequence per length (optionally pre-filled with `starts` positions) and
    plans a step of `lens` new tokens each.  Returns (ctx, slots)."""
    from gguf_rs_cli_b200.engine.step import Entry
    slots = [eng.open() for _ in lens]
    if starts:
        eng.cache.reserve(slots, starts)
        eng.cache.advance(slots, starts)
    ctx, _, _ = eng.plan([Entry(s, [1] * n, ()) for s, n in zip(slots, lens)])
    return ctx, slots


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_embedding_norm_head_alone(name, dtype):
    from gguf_rs_cli_b200.parts.base import Stream
    cfg, w, model = config(name), plain_weights(name), llm(name, dtype).model
    eng = new_engine(name, dtype)
    ctx, _ = plan_for(eng, [7, 3])
    toks = torch.tensor(tokens_of(name, 10, 1), dtype=torch.int32, device=DEV)
    x = model.embedding.forward(toks, ctx)
    want_x = P.embedding(w["model.embed_tokens.weight"], toks.tolist())
    assert torch.equal(x.cpu(), want_x)
    # norm folds a pending term into the stream in 32-bit
    pend = (torch.randn(10, cfg["hidden_size"]) * 0.1).to(tdtype(dtype))
    stream = Stream(x.clone())
    stream.pending = pend.to(DEV)
    norm = model.layers[0].norms["mixer"]
    h = norm.apply(stream, ctx)
    want = P.rmsnorm(want_x + pend.float(), w["model.layers.0.input_layernorm.weight"], cfg["rms_norm_eps"])
    assert_close(h, want, dtype, "norm")
    assert stream.pending is None and torch.allclose(stream.x.cpu(), want_x + pend.float(), atol=1e-6)
    # head on gathered rows
    rows = torch.tensor([9, 2], dtype=torch.int32, device=DEV)
    hf = model.final_norm.apply(stream, ctx, rows=rows, buffer="t.final")
    logits = model.head.forward(hf, ctx)
    head_w = w.get("lm_head.weight", w["model.embed_tokens.weight"])
    want_l = P.linear(P.rmsnorm((want_x + pend.float())[[9, 2]], w["model.norm.weight"], cfg["rms_norm_eps"]), head_w)
    assert logits.dtype == torch.float32
    assert_close(logits, want_l, dtype, "head")


def test_rotary_tables():
    from gguf_rs_cli_b200.config.specs import PartSpec
    from gguf_rs_cli_b200.parts.rotary import Rotary
    for name in "ABC":
        cfg = config(name)
        model = llm(name, "float32").model
        (rot,) = model.positions.values()                      # one table shared by all layers
        assert torch.equal(rot.inv_freq.cpu(), P.inv_freq_table(cfg))
    lin = Rotary(PartSpec("rope", dict(head_dim=32, rotary_dim=16, theta=100.0, pairing="interleaved",
                                       scaling={"rope_type": "linear", "factor": 4.0})), torch.float32, DEV)
    want = torch.tensor([100.0 ** (-2 * i / 16) / 4 for i in range(8)])
    assert torch.allclose(lin.inv_freq.cpu(), want) and lin.pairing == 1 and lin.rotary_dim == 16
    with pytest.raises(ValueError, match="rotary_dim"):
        Rotary(PartSpec("rope", dict(head_dim=32, rotary_dim=34, theta=1.0)), torch.float32, DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_attention_and_feed_forward_alone(name, dtype):
    cfg, w, model = config(name), plain_weights(name), llm(name, dtype).model
    E, nh, nkv, hd = cfg["hidden_size"], cfg["num_attention_heads"], P.kv_heads_of(cfg), P.head_dim_of(cfg)
    eng = new_engine(name, dtype)
    lens = [70, 5]
    ctx, slots = plan_for(eng, lens)
    g = torch.Generator().manual_seed(3)
    h = torch.randn(sum(lens), E, generator=g).to(tdtype(dtype))
    layer, p = model.layers[1], "model.layers.1."
    run = eng.runs[1]
    got = layer.mixer.forward(h.to(DEV), ctx, run)
    inv = P.inv_freq_table(cfg)
    # a part that took the weight of the norm in front of it into its matrix expects rows without it
    wn_m = w[p + "input_layernorm.weight"] if layer.block.absorbed["mixer"] else 1.0
    wn_f = w[p + "post_attention_layernorm.weight"] if layer.block.absorbed["feed_forward"] else 1.0
    assert layer.block.absorbed["mixer"] == layer.block.absorbed["feed_forward"] == (dtype == "bfloat16")
    want, t0 = [], 0
    for n in lens:
        hh = h[t0:t0 + n].float() * wn_m
        q = P.linear(hh, w[p + "self_attn.q_proj.weight"], w.get(p + "self_attn.q_proj.bias")).reshape(n, nh, hd)
        k = P.linear(hh, w[p + "self_attn.k_proj.weight"], w.get(p + "self_attn.k_proj.bias")).reshape(n, nkv, hd)
        v = P.linear(hh, w[p + "self_attn.v_proj.weight"], w.get(p + "self_attn.v_proj.bias")).reshape(n, nkv, hd)
        pos = torch.arange(n)
        a = P.attention(P.rope(q, pos, inv), P.rope(k, pos, inv), v)
        want.append(P.linear(a, w[p + "self_attn.o_proj.weight"]))
        t0 += n
    assert_close(got, torch.cat(want), dtype, "attention part")
    got_ff = layer.feed_forward.forward(h.to(DEV), ctx)
    want_ff = P.feed_forward(h.float() * wn_f, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                             w[p + "mlp.down_proj.weight"])
    assert_close(got_ff, want_ff, dtype, "feed-forward part")


# ------------------------------------------------------------------ toy parts
def register_toys():
    """A mixer with fixed-size state of its own (the running mean of its inputs, then a
    projection), written with torch here and registered from here: nothing in the package
    knows it."""
    from gguf_rs_cli_b200.config import register_architecture
    from gguf_rs_cli_b200.config.llama import LlamaConfig, build_llama_spec
    from gguf_rs_cli_b200.config.specs import LayerSpec, ModelSpec, PartSpec, Run
    from gguf_rs_cli_b200.parts import MIXERS, Part, register_mixer
    from gguf_rs_cli_b200.weights import TensorRequest
    if "running_mean" in MIXERS.kinds():
        return

    @register_mixer("running_mean")
    class RunningMean(Part):
        def __init__(self, spec, dtype, device, position=None):
            super().__init__(spec, dtype, device)

        def kv_spec(self):
            return None

        def state_spec(self):
            return {"sum": ((self.p["hidden_size"],), "float32"), "count": ((), "float32")}

        def tensor_requests(self):
            E = self.p["hidden_size"]
            return [TensorRequest(self.spec.tensors["proj"], (E, E))]

        def load(self, store):
            self.proj = store.get(self.tensor_requests()[0])

        def forward(self, h, ctx, run):
            total, count = ctx.state(f"run{run.index}.sum"), ctx.state(f"run{run.index}.count")
            out = torch.zeros(h.shape, dtype=torch.float32, device=h.device)
            t0 = 0
            for slot, n in zip(ctx.host["slots"], ctx.host["qlens"]):
                cs = h[t0:t0 + n].float().cumsum(0) + total[slot]
                cnt = count[slot] + torch.arange(1, n + 1, device=h.device, dtype=torch.float32)
                out[t0:t0 + n] = cs / cnt[:, None]
                total[slot] = cs[-1]
                count[slot] = cnt[-1]
                t0 += n
            return (out @ self.proj.float().t()).to(ctx.dtype)

    @dataclass(frozen=True)
    class ToyConfig:
        llama: LlamaConfig
        window: int

        @classmethod
        def from_dict(cls, raw):
            return cls(LlamaConfig.from_dict(raw), int(raw.get("toy_window", 0)))

    def build_toy_spec(cfg: ToyConfig) -> ModelSpec:
        """Layer 0: windowed attention.  Layer 1: the running-mean mixer.  Layer 2: attention
        over all keys.  Layer 3: attention without k/v of its own, reading layer 2's cache.
        Run order: 0, 1, 2, 3, then layer 0 again (its second run has a cache of its own)."""
        base = build_llama_spec(cfg.llama)
        E = cfg.llama.hidden_size
        layers = []
        for i, ls in enumerate(base.layers):
            mixer = ls.mixer
            if i == 0:
                mixer = PartSpec("attention", {**mixer.params, "window": cfg.window}, mixer.tensors)
            elif i == 1:
                mixer = PartSpec("running_mean", {"hidden_size": E}, {"proj": f"model.layers.{i}.mean.proj.weight"})
            elif i == 3:
                t = {k: v for k, v in mixer.tensors.items() if k in ("q", "o")}
                mixer = PartSpec("attention", {**mixer.params, "shares_kv": True}, t)
            layers.append(LayerSpec(ls.block, mixer, ls.feed_forward, ls.norms, ls.position))
        return ModelSpec(**{**base.__dict__, "architecture": "ToyForCausalLM", "layers": layers,
                            "schedule": [Run(0), Run(1), Run(2), Run(3, cache_of=2), Run(0)]})

    register_architecture("ToyForCausalLM", ToyConfig, build_toy_spec)


TOY = {**config("A"), "architectures": ["ToyForCausalLM"], "model_type": "toy", "num_hidden_layers": 4, "toy_window": 70,
       "max_position_embeddings": 512}


def toy_weights(seed=0):
    cfg = {**TOY, "architectures": ["LlamaForCausalLM"]}
    w = P.random_weights(cfg, seed, std=0.05, norm_noise=0.1)
    for n in ("q_proj", "k_proj", "v_proj", "o_proj"):
        del w[f"model.layers.1.self_attn.{n}.weight"]
    for n in ("k_proj", "v_proj"):
        del w[f"model.layers.3.self_attn.{n}.weight"]
    g = torch.Generator().manual_seed(seed + 1)
    w["model.layers.1.mean.proj.weight"] = torch.randn(64, 64, generator=g) * 0.05
    return {k: v.to(torch.bfloat16).float() for k, v in w.items()}


def toy_plain_forward(w, tokens):
    """The toy model on one whole sequence, from the plain parts."""
    cfg = TOY
    nh, nkv, hd, eps = 4, 2, 16, cfg["rms_norm_eps"]
    T = len(tokens)
    pos, inv = torch.arange(T), P.inv_freq_table(cfg)
    x = P.embedding(w["model.embed_tokens.weight"], tokens)
    kv2 = None
    for run, l in enumerate([0, 1, 2, 3, 0]):
        p = f"model.layers.{l}."
        xn = P.rmsnorm(x, w[p + "input_layernorm.weight"], eps)
        if l == 1:
            mean = xn.cumsum(0) / torch.arange(1, T + 1)[:, None]
            x = x + P.linear(mean, w[p + "mean.proj.weight"])
        else:
            q = P.rope(P.linear(xn, w[p + "self_attn.q_proj.weight"]).reshape(T, nh, hd), pos, inv)
            if l == 3:
                k, v = kv2
            else:
                k = P.rope(P.linear(xn, w[p + "self_attn.k_proj.weight"]).reshape(T, nkv, hd), pos, inv)
                v = P.linear(xn, w[p + "self_attn.v_proj.weight"]).reshape(T, nkv, hd)
            if l == 2:
                kv2 = (k, v)
            a = P.attention(q, k, v, window=cfg["toy_window"] if l == 0 else None)
            x = x + P.linear(a, w[p + "self_attn.o_proj.weight"])
        xn = P.rmsnorm(x, w[p + "post_attention_layernorm.weight"], eps)
        x = x + P.feed_forward(xn, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    x = P.rmsnorm(x, w["model.norm.weight"], eps)
    return P.linear(x, w["lm_head.weight"])


@pytest.mark.parametrize("dtype", DTYPES)
def test_toy_architecture_with_state_window_shared_cache_and_a_layer_run_twice(dtype):
    from gguf_rs_cli_b200.api import _build
    from gguf_rs_cli_b200.engine.step import Engine, Entry
    from gguf_rs_cli_b200.weights import TensorSource
    register_toys()
    w = toy_weights()
    model = _build(dict(TOY), TensorSource(tensors={k: v.to(torch.bfloat16) for k, v in w.items()}, where="toy"),
                   dtype, DEV).model
    eng = Engine(model, n_tokens=64 * 24, n_slots=3, max_len=512, max_step_tokens=128)
    # the cache has a windowed group (runs 0 and 4), a full group (run 2), and run 3 reads run 2's
    kinds = {(g.spec.window, tuple(g.runs)) for g in eng.cache.groups}
    assert kinds == {(70, (0, 4)), (None, (2,))}
    assert eng.runs[3].k.data_ptr() == eng.runs[2].k.data_ptr() and not eng.runs[3].owns_cache
    assert "run1.sum" in eng.cache.states and eng.runs[1].k is None
    ring = [g for g in eng.cache.groups if g.spec.window][0].ring_pages
    assert ring == 5                                       # 70 + 128 - 1 positions and one page of slack

    g = torch.Generator().manual_seed(9)
    seqs = [torch.randint(0, 256, (n,), generator=g).tolist() for n in (300, 150, 40)]
    want = [toy_plain_forward(w, s) for s in seqs]
    # two batches over the same slots; pieces of unequal lengths, then single tokens; shorter ones end earlier
    for rnd in range(2):
        slots = [eng.open() for _ in seqs]
        fed = [0] * len(seqs)
        live = list(range(len(seqs)))
        pieces = [[100, 1], [128, 7], [20, 5]]
        while live:
            entries, idx = [], []
            for i in live:
                n = pieces[i].pop(0) if pieces[i] else (1 if fed[i] > len(seqs[i]) - 12 else 31)
                n = min(n, len(seqs[i]) - fed[i])
                entries.append(Entry(slots[i], seqs[i][fed[i]:fed[i] + n], range(n)))
                idx.append((i, n))
            logits = eng.step(entries)
            row = 0
            for i, n in idx:
                assert_close(logits[row:row + n], want[i][fed[i]:fed[i] + n], dtype, f"round {rnd} seq {i} at {fed[i]}")
                row += n
                fed[i] += n
            for i in list(live):
                if fed[i] == len(seqs[i]):
                    eng.close(slots[i])
                    live.remove(i)
        eng.cache.check()
        assert eng.cache.slots.held_count == 0 and all(g.pool.held_count == 0 for g in eng.cache.groups)


def test_schedule_errors_are_found_when_the_model_is_built():
    from gguf_rs_cli_b200.config import load_config
    from gguf_rs_cli_b200.config.specs import ModelSpec, Run
    from gguf_rs_cli_b200.models import Decoder
    register_toys()
    arch, cfg = load_config(dict(TOY))
    spec = arch.build_spec(cfg)
    bad = ModelSpec(**{**spec.__dict__, "schedule": [Run(0), Run(1), Run(2), Run(3)]})       # layer 3 has no k/v and no source
    with pytest.raises(ValueError, match="cache_of"):
        Decoder(bad, torch.float32, "meta")
    bad = ModelSpec(**{**spec.__dict__, "schedule": [Run(0), Run(1), Run(2), Run(0, cache_of=2)]})
    with pytest.raises(ValueError, match="of its own"):
        Decoder(bad, torch.float32, "meta")
    bad = ModelSpec(**{**spec.__dict__, "schedule": [Run(0), Run(1), Run(2), Run(3, cache_of=0)]})  # window != all keys
    with pytest.raises(ValueError, match="does not match"):
        Decoder(bad, torch.float32, "meta")


# ------------------------------- a routed feed-forward and another position encoding
def register_more_toys():
    """Two more kinds registered from here: a feed-forward that routes every token to one of a few small experts
    (router logits in 32-bit, top-1, the winner's gated MLP scaled by its softmax weight), and a position
    encoding of its own (interleaved pairs over half of each head, frequencies that fall off linearly).  An
    architecture uses them in alternate layers beside the library's own parts."""
    from gguf_rs_cli_b200.config import register_architecture
    from gguf_rs_cli_b200.config.llama import LlamaConfig, build_llama_spec
    from gguf_rs_cli_b200.config.specs import LayerSpec, ModelSpec, PartSpec, Run
    from gguf_rs_cli_b200.parts import FEED_FORWARDS, Part, register_feed_forward, register_position
    from gguf_rs_cli_b200.weights import TensorRequest
    if "top1_experts" in FEED_FORWARDS.kinds():
        return

    @register_feed_forward("top1_experts")
    class Top1Experts(Part):
        def tensor_requests(self):
            E, F, n, t = self.p["hidden_size"], self.p["expert_size"], self.p["experts"], self.spec.tensors
            return [TensorRequest(t["router"], (n, E)), TensorRequest(t["gate"], (n, F, E)), TensorRequest(t["up"], (n, F, E)),
                    TensorRequest(t["down"], (n, E, F))]

        def load(self, store):
            self.router, self.gate, self.up, self.down = (store.get(r).float() for r in self.tensor_requests())

        def forward(self, h, ctx):
            x = h.float()
            weight = torch.softmax(x @ self.router.t(), dim=-1)                 # [T, experts], 32-bit
            best = weight.argmax(-1)
            out = torch.zeros_like(x)
            for e in range(self.p["experts"]):
                rows = (best == e).nonzero().flatten()
                if rows.numel():
                    xe = x[rows]
                    a = torch.nn.functional.silu(xe @ self.gate[e].t()) * (xe @ self.up[e].t())
                    out[rows] = (a @ self.down[e].t()) * weight[rows, e:e + 1]
            return out.to(ctx.dtype)

    @register_position("linear_interleaved")
    class LinearInterleaved(Part):
        def __init__(self, spec, dtype, device):
            super().__init__(spec, dtype, device)
            self.rotary_dim = self.p["head_dim"] // 2
            self.pairing = 1
            n = self.rotary_dim // 2
            self.inv_freq = torch.tensor([self.p["top"] * (1.0 - i / n) for i in range(n)], dtype=torch.float32, device=device)

    @dataclass(frozen=True)
    class Toy2Config:
        llama: LlamaConfig
        experts: int
        expert_size: int
        top: float

        @classmethod
        def from_dict(cls, raw):
            return cls(LlamaConfig.from_dict(raw), int(raw["toy_experts"]), int(raw["toy_expert_size"]), float(raw["toy_top_frequency"]))

    def build_toy2_spec(cfg: Toy2Config) -> ModelSpec:
        """Odd layers: routed experts instead of the dense feed-forward.  Even layers: the new position encoding."""
        base = build_llama_spec(cfg.llama)
        E, hd = cfg.llama.hidden_size, cfg.llama.head_dim
        layers = []
        for i, ls in enumerate(base.layers):
            ff, position = ls.feed_forward, ls.position
            if i % 2 == 1:
                p = f"model.layers.{i}.experts."
                ff = PartSpec("top1_experts", {"hidden_size": E, "experts": cfg.experts, "expert_size": cfg.expert_size},
                              {"router": p + "router.weight", "gate": p + "gate.weight", "up": p + "up.weight", "down": p + "down.weight"})
            else:
                position = PartSpec("linear_interleaved", {"head_dim": hd, "top": cfg.top}, {})
            layers.append(LayerSpec(ls.block, ls.mixer, ff, ls.norms, position))
        return ModelSpec(**{**base.__dict__, "architecture": "Toy2ForCausalLM", "layers": layers})

    register_architecture("Toy2ForCausalLM", Toy2Config, build_toy2_spec)


TOY2 = {**config("B"), "architectures": ["Toy2ForCausalLM"], "model_type": "toy2", "num_hidden_layers": 4, "toy_experts": 3,
        "toy_expert_size": 40, "toy_top_frequency": 0.7}


def toy2_weights(seed=0):
    cfg = {**TOY2, "architectures": ["LlamaForCausalLM"]}
    w = P.random_weights(cfg, seed, std=0.05, norm_noise=0.1)
    E, n, F = cfg["hidden_size"], TOY2["toy_experts"], TOY2["toy_expert_size"]
    g = torch.Generator().manual_seed(seed + 7)
    for i in (1, 3):
        for name in ("gate_proj", "up_proj", "down_proj"):
            del w[f"model.layers.{i}.mlp.{name}.weight"]
        p = f"model.layers.{i}.experts."
        w[p + "router.weight"] = torch.randn(n, E, generator=g) * 0.5
        w[p + "gate.weight"] = torch.randn(n, F, E, generator=g) * 0.05
        w[p + "up.weight"] = torch.randn(n, F, E, generator=g) * 0.05
        w[p + "down.weight"] = torch.randn(n, E, F, generator=g) * 0.05
    return {k: v.to(torch.bfloat16).float() for k, v in w.items()}


def toy2_plain_forward(w, tokens):
    cfg = TOY2
    nh, nkv, hd, eps = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["rms_norm_eps"]
    T = len(tokens)
    pos = torch.arange(T)
    x = P.embedding(w["model.embed_tokens.weight"], tokens)

    def rotate(t, layer):
        if layer % 2 == 1:
            return P.rope(t, pos, P.inv_freq_table(cfg))
        rd = hd // 2
        f = torch.tensor([cfg["toy_top_frequency"] * (1.0 - i / (rd // 2)) for i in range(rd // 2)])
        ang = pos[:, None].float() * f[None, :]
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        out = t.clone()
        a, b = t[..., 0:rd:2], t[..., 1:rd:2]                       # pairs (2i, 2i+1) of the first half of the head
        out[..., 0:rd:2], out[..., 1:rd:2] = a * c - b * s, a * s + b * c
        return out

    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        xn = P.rmsnorm(x, w[p + "input_layernorm.weight"], eps)
        proj = lambda n: P.linear(xn, w[p + f"self_attn.{n}_proj.weight"], w.get(p + f"self_attn.{n}_proj.bias"))
        q = rotate(proj("q").reshape(T, nh, hd), l)
        k = rotate(proj("k").reshape(T, nkv, hd), l)
        v = proj("v").reshape(T, nkv, hd)
        x = x + P.linear(P.attention(q, k, v), w[p + "self_attn.o_proj.weight"])
        xn = P.rmsnorm(x, w[p + "post_attention_layernorm.weight"], eps)
        if l % 2 == 1:
            e = p + "experts."
            weight = P.softmax(P.linear(xn, w[e + "router.weight"]))
            best = weight.argmax(-1)
            term = torch.zeros_like(x)
            for t in range(T):
                i = int(best[t])
                term[t] = P.feed_forward(xn[t:t + 1], w[e + "gate.weight"][i], w[e + "up.weight"][i], w[e + "down.weight"][i])[0] * weight[t, i]
            x = x + term
        else:
            x = x + P.feed_forward(xn, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    x = P.rmsnorm(x, w["model.norm.weight"], eps)
    return P.linear(x, w.get("lm_head.weight", w["model.embed_tokens.weight"]))


def test_toy_architecture_with_routed_experts_and_a_position_encoding_of_its_own():
    """Registered, built and stepped without a change to the package: whole prompts, then token by token with
    unequal lengths, against the plain formulas.  32-bit (the winner of a near-tied router would differ between
    roundings in bfloat16)."""
    from gguf_rs_cli_b200.api import _build
    from gguf_rs_cli_b200.engine.step import Engine, Entry
    from gguf_rs_cli_b200.weights import TensorSource
    register_more_toys()
    w = toy2_weights()
    model = _build(dict(TOY2), TensorSource(tensors={k: v.to(torch.bfloat16) for k, v in w.items()}, where="toy2"),
                   "float32", DEV).model
    kinds = [(type(l.feed_forward).__name__, type(l.mixer.position).__name__) for l in model.layers]
    assert kinds == [("GatedMLP", "LinearInterleaved"), ("Top1Experts", "Rotary")] * 2
    eng = Engine(model, n_tokens=64 * 8, n_slots=2, max_len=256)
    g = torch.Generator().manual_seed(4)
    seqs = [torch.randint(0, TOY2["vocab_size"], (n,), generator=g).tolist() for n in (90, 37)]
    want = [toy2_plain_forward(w, s) for s in seqs]
    slots = [eng.open() for _ in seqs]
    cut = [70, 20]
    logits = eng.step([Entry(s, q[:c], range(c)) for s, q, c in zip(slots, seqs, cut)])
    assert_close(logits[:70], want[0][:70], "float32", "prompt 0")
    assert_close(logits[70:], want[1][:20], "float32", "prompt 1")
    for step in range(20):
        live = [i for i in range(2) if cut[i] + step < len(seqs[i])]
        logits = eng.step([Entry(slots[i], [seqs[i][cut[i] + step]], [0]) for i in live])
        for row, i in enumerate(live):
            assert_close(logits[row:row + 1], want[i][cut[i] + step:cut[i] + step + 1], "float32", f"seq {i} token {cut[i] + step}")
    for s in slots:
        eng.close(s)
    eng.cache.check()


# ------------------------------------------ hooks: planning on the host, and whether a step may be captured
def test_a_mixer_without_hooks_generates_under_captured_graphs_untouched():
    """The running-mean mixer above computes with host values every step and says nothing about CUDA graphs:
    the backend then never captures a step that contains it, and generation with graphs switched on gives
    the plain result."""
    from gguf_rs_cli_b200.api import _build
    from gguf_rs_cli_b200.engine.backend import EngineBackend
    from gguf_rs_cli_b200.engine.generate import generate_ids
    from gguf_rs_cli_b200.engine.step import Engine
    from gguf_rs_cli_b200.sampling import SamplingParams
    from gguf_rs_cli_b200.weights import TensorSource
    register_toys()
    w = toy_weights()
    model = _build(dict(TOY), TensorSource(tensors={k: v.to(torch.bfloat16) for k, v in w.items()}, where="toy"),
                   "float32", DEV).model
    assert not model.capturable
    g = torch.Generator().manual_seed(21)
    prompts = [torch.randint(0, 256, (n,), generator=g).tolist() for n in (9, 30)]
    want = []
    for p in prompts:
        seq = list(p)
        for _ in range(6):
            seq.append(int(toy_plain_forward(w, seq)[-1].argmax()))
        want.append(seq[len(p):])
    backend = EngineBackend(Engine(model, n_tokens=64 * 8, n_slots=2, max_len=512, max_step_tokens=128), use_graphs=True)
    assert generate_ids(backend, prompts, 6, SamplingParams(temperature=0.0), []) == want
    assert backend._graphs == {}


def register_shift_toy():
    """A mixer that plans on the host and may be captured: it adds a projection of the row in front of each token
    (the last row of the step before for a sequence's first token, kept as fixed-size state).  Which row that
    is, and where each sequence's last row lies, it lays out on the host in `plan`; the arrays travel with the
    step's own index arrays.  Its graph class is the number of sequences, which fixes the arrays' sizes."""
    from gguf_rs_cli_b200.config import register_architecture
    from gguf_rs_cli_b200.config.llama import LlamaConfig, build_llama_spec
    from gguf_rs_cli_b200.config.specs import LayerSpec, ModelSpec, PartSpec
    from gguf_rs_cli_b200.parts import MIXERS, Part, register_mixer
    from gguf_rs_cli_b200.weights import TensorRequest
    if "shift" in MIXERS.kinds():
        return

    @register_mixer("shift")
    class Shift(Part):
        def __init__(self, spec, dtype, device, position=None):
            super().__init__(spec, dtype, device)

        def kv_spec(self):
            return None

        def state_spec(self):
            return {"last": ((self.p["hidden_size"],), "float32")}

        def tensor_requests(self):
            E = self.p["hidden_size"]
            return [TensorRequest(self.spec.tensors["proj"], (E, E))]

        def load(self, store):
            self.proj = store.get(self.tensor_requests()[0]).float()

        def plan(self, batch):
            prev, last, t0 = [], [], 0
            for n in batch.qlens:
                prev += [-1] + list(range(t0, t0 + n - 1))
                t0 += n
                last.append(t0 - 1)
            return {"prev": prev, "last": last}

        def graph_class(self, batch):
            return len(batch.slots)

        def forward(self, h, ctx, run):
            plan = ctx.plan_of(self)
            prev, last = plan["prev"].long(), plan["last"].long()
            n_tok, n_seq = prev.numel(), last.numel()             # real tokens and sequences (the rest is padding)
            state = ctx.state(f"run{run.index}.last")
            slots = ctx.slots[:n_seq].long()
            hf = h[:n_tok].float()
            before = state[slots][ctx.seq_of[:n_tok].long()]       # what each token's sequence left behind
            rows = torch.where((prev < 0)[:, None], before, hf[prev.clamp(min=0)])
            state.index_copy_(0, slots, hf[last])
            out = torch.zeros(h.shape, dtype=torch.float32, device=h.device)
            out[:n_tok] = rows @ self.proj.t()
            return out.to(ctx.dtype)

    @dataclass(frozen=True)
    class ShiftConfig:
        llama: LlamaConfig

        @classmethod
        def from_dict(cls, raw):
            return cls(LlamaConfig.from_dict(raw))

    def build_shift_spec(cfg: ShiftConfig) -> ModelSpec:
        base = build_llama_spec(cfg.llama)
        layers = list(base.layers)
        ls = layers[1]
        layers[1] = LayerSpec(ls.block, PartSpec("shift", {"hidden_size": cfg.llama.hidden_size},
                                                 {"proj": "model.layers.1.shift.proj.weight"}), ls.feed_forward, ls.norms, None)
        return ModelSpec(**{**base.__dict__, "architecture": "ShiftForCausalLM", "layers": layers})

    register_architecture("ShiftForCausalLM", ShiftConfig, build_shift_spec)


def test_a_mixer_that_plans_on_the_host_is_captured_and_replanned_every_step():
    from gguf_rs_cli_b200.api import _build
    from gguf_rs_cli_b200.engine.backend import EngineBackend
    from gguf_rs_cli_b200.engine.generate import generate_ids
    from gguf_rs_cli_b200.engine.step import Engine
    from gguf_rs_cli_b200.sampling import SamplingParams
    from gguf_rs_cli_b200.weights import TensorSource
    register_shift_toy()
    raw = {**config("A"), "architectures": ["ShiftForCausalLM"], "model_type": "shift", "num_hidden_layers": 3}
    w = P.random_weights({**raw, "architectures": ["LlamaForCausalLM"]}, 5, std=0.05, norm_noise=0.1)
    for n in ("q_proj", "k_proj", "v_proj", "o_proj"):
        del w[f"model.layers.1.self_attn.{n}.weight"]
    w["model.layers.1.shift.proj.weight"] = torch.randn(64, 64, generator=torch.Generator().manual_seed(6)) * 0.3
    w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}

    def plain(tokens):
        T, eps, inv = len(tokens), raw["rms_norm_eps"], P.inv_freq_table(raw)
        x = P.embedding(w["model.embed_tokens.weight"], tokens)
        for l in range(3):
            p = f"model.layers.{l}."
            xn = P.rmsnorm(x, w[p + "input_layernorm.weight"], eps)
            if l == 1:
                shifted = torch.cat([torch.zeros(1, 64), xn[:-1]])
                x = x + P.linear(shifted, w[p + "shift.proj.weight"])
            else:
                x = P.layer(raw, w, l, x, torch.arange(T), inv)            # a whole plain layer
                continue
            xn = P.rmsnorm(x, w[p + "post_attention_layernorm.weight"], eps)
            x = x + P.feed_forward(xn, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
        return P.linear(P.rmsnorm(x, w["model.norm.weight"], eps), w["lm_head.weight"])

    model = _build(raw, TensorSource(tensors={k: v.to(torch.bfloat16) for k, v in w.items()}, where="shift"), "float32", DEV).model
    assert model.capturable and len(model.planners) == 2          # the attention layers share one plan, the toy has its own
    g = torch.Generator().manual_seed(8)
    prompts = [torch.randint(0, 256, (n,), generator=g).tolist() for n in (7, 66, 20)]
    want = []
    for p in prompts:
        seq = list(p)
        for _ in range(8):
            seq.append(int(plain(seq)[-1].argmax()))
        want.append(seq[len(p):])
    for graphs in (False, True):
        backend = EngineBackend(Engine(model, n_tokens=64 * 8, n_slots=4, max_len=128), use_graphs=graphs)
        for _ in range(2):                                          # the second batch uses the slots, and the graphs, again
            assert generate_ids(backend, prompts, 8, SamplingParams(temperature=0.0), []) == want
        if graphs:
            captured = [dg for dg in backend._graphs.values() if dg.graph is not None]
            assert captured and all(dg.plan_words == 2 * 3 for dg in captured)
            assert {key[1][-1] for key in backend._graphs} == {3}  # the toy's class is part of every graph's key

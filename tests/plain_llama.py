"""Plain, slow Llama decoder used as the oracle of every test.

It rests on the formulas of the reference's CPU forward pass (the reference is a
Rust program and cannot be compiled or imported here, so nothing below was checked
against a run of it; each function cites the lines it restates).  Whole sequences,
no cache, one function for each part, torch on the CPU, and no code shared with the
package under test: the configuration is a plain dict of config.json keys and the
weights a plain dict of tensors under their safetensors names.

The llama3 frequency rule and the sampling walk in index order are not in the
reference; they are stated in the docstrings of `inv_freq_table` and `sample`.
"""
import math

import torch


# --------------------------------------------------------------------- config
def head_dim_of(cfg):
    """head_dim = n_embd / n_heads unless config.json gives one (src/model/config.rs:48)."""
    hd = cfg.get("head_dim")
    return int(hd) if hd else cfg["hidden_size"] // cfg["num_attention_heads"]


def kv_heads_of(cfg):
    """n_kv_heads defaults to n_heads (src/model/config.rs:35)."""
    n = cfg.get("num_key_value_heads")
    return int(n) if n else cfg["num_attention_heads"]


# ---------------------------------------------------------------------- parts
def embedding(table, tokens):
    """x = E_tok[token, :] (src/model/llama.rs:349, src/tensor/dequant.rs:270-274)."""
    return table[torch.as_tensor(tokens, dtype=torch.long)]


def rmsnorm(x, w, eps):
    """rms = sqrt(sum(x^2)/n + eps); x = x / rms * w (src/math/ops.rs:1-4)."""
    rms = torch.sqrt((x * x).sum(-1, keepdim=True) / x.shape[-1] + eps)
    return x / rms * w


def linear(x, w, b=None):
    """y[i] = sum_j W[i,j] x[j], W row-major [out, in] (src/tensor/dequant.rs:315-317);
    optional bias added after (src/model/llama.rs:367-369)."""
    y = x @ w.t()
    return y if b is None else y + b


def inv_freq_table(cfg, dtype=torch.float32):
    """f_i = base^(-2i/hd) for i < hd/2 (src/math/rope.rs:8).

    llama3 scaling (not in the reference): with wavelength l = 2*pi/f_i and the keys
    factor, low_freq_factor, high_freq_factor, original_max_position_embeddings (orig):
    l < orig/high keeps f_i; l > orig/low gives f_i/factor; between them
    s = (orig/l - low)/(high - low) and f_i = (1-s)*f_i/factor + s*f_i.
    "linear" scaling divides every f_i by factor.  Built in 64-bit, returned in 32-bit.
    """
    hd = head_dim_of(cfg)
    base = float(cfg.get("rope_theta", 10000.0))
    idx = torch.arange(0, hd // 2, dtype=torch.float64)
    f = base ** (-2.0 * idx / hd)
    sc = cfg.get("rope_scaling")
    kind = None if not sc else sc.get("rope_type", sc.get("type"))
    if kind == "llama3":
        factor = float(sc["factor"])
        low = float(sc["low_freq_factor"])
        high = float(sc["high_freq_factor"])
        orig = float(sc["original_max_position_embeddings"])
        out = []
        for fi in f.tolist():
            lam = 2.0 * math.pi / fi
            if lam < orig / high:
                out.append(fi)
            elif lam > orig / low:
                out.append(fi / factor)
            else:
                s = (orig / lam - low) / (high - low)
                out.append((1.0 - s) * fi / factor + s * fi)
        f = torch.tensor(out, dtype=torch.float64)
    elif kind == "linear":
        f = f / float(sc["factor"])
    elif kind not in (None, "default"):
        raise ValueError(f"plain reference: rope scaling {kind!r}")
    return f.to(torch.float32).to(dtype)


def rope(x, positions, inv_freq):
    """Half-split rotation of every head: pairs (i, i+hd/2), angle pos*f_i
    (src/math/rope.rs:6-13).  x: [T, heads, hd]; positions: [T]."""
    half = x.shape[-1] // 2
    ang = positions.to(inv_freq.dtype)[:, None] * inv_freq[None, :]     # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    x0, x1 = x[..., :half], x[..., half:]
    return torch.cat([x0 * c - x1 * s, x0 * s + x1 * c], dim=-1)


def softmax(s):
    """exp(s - max) / sum (src/math/ops.rs:5-10)."""
    m = s.max(-1, keepdim=True).values
    e = torch.exp(s - m)
    return e / e.sum(-1, keepdim=True)


def attention(q, k, v, window=None):
    """Causal grouped attention of one whole sequence (src/model/llama.rs:374-394):
    query head h reads KV head h // (nh/nkv); scores q.k / sqrt(hd) over positions
    <= its own (and, with a window W, > pos - W: not in the reference); softmax;
    weighted sum of values.  q: [T, nh, hd]; k, v: [T, nkv, hd] -> [T, nh*hd]."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    ratio = nh // nkv
    out = torch.zeros(T, nh, hd, dtype=q.dtype)
    scale = math.sqrt(hd)
    for h in range(nh):
        g = h // ratio
        s = (q[:, h, :] @ k[:, g, :].t()) / scale                        # [T, T]
        i = torch.arange(T)
        mask = i[None, :] > i[:, None]
        if window:
            mask = mask | (i[None, :] <= i[:, None] - window)
        s = s.masked_fill(mask, float("-inf"))
        out[:, h, :] = softmax(s) @ v[:, g, :]
    return out.reshape(T, nh * hd)


def silu(x):
    """x / (1 + exp(-x)) (src/math/ops.rs:11)."""
    return x / (1.0 + torch.exp(-x))


def feed_forward(xn, wg, wu, wd):
    """down(silu(gate(xn)) * up(xn)) (src/model/llama.rs:399-402)."""
    return linear(silu(linear(xn, wg)) * linear(xn, wu), wd)


# ---------------------------------------------------------------------- model
def layer(cfg, w, l, x, positions, inv_freq):
    """One decoder layer on a whole sequence (src/model/llama.rs:361-404):
    norm, Q/K/V (+bias before the rotation), rotation of q and k, attention, output
    projection added to x, norm, feed-forward added to x."""
    p = f"model.layers.{l}."
    nh, nkv, hd = cfg["num_attention_heads"], kv_heads_of(cfg), head_dim_of(cfg)
    eps = float(cfg.get("rms_norm_eps", 1e-6))
    T = x.shape[0]
    xn = rmsnorm(x, w[p + "input_layernorm.weight"], eps)
    q = linear(xn, w[p + "self_attn.q_proj.weight"], w.get(p + "self_attn.q_proj.bias"))
    k = linear(xn, w[p + "self_attn.k_proj.weight"], w.get(p + "self_attn.k_proj.bias"))
    v = linear(xn, w[p + "self_attn.v_proj.weight"], w.get(p + "self_attn.v_proj.bias"))
    q = rope(q.reshape(T, nh, hd), positions, inv_freq)
    k = rope(k.reshape(T, nkv, hd), positions, inv_freq)
    a = attention(q, k, v.reshape(T, nkv, hd))
    x = x + linear(a, w[p + "self_attn.o_proj.weight"])
    xn = rmsnorm(x, w[p + "post_attention_layernorm.weight"], eps)
    x = x + feed_forward(xn, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                         w[p + "mlp.down_proj.weight"])
    return x


def forward(cfg, w, tokens, dtype=torch.float32):
    """Logits [T, V] at every position of one whole sequence
    (src/model/llama.rs:343-409; the head falls back to the embedding table when
    there is no output matrix, src/model/llama.rs:124)."""
    w = {k: v.to(dtype) for k, v in w.items()}
    positions = torch.arange(len(tokens))
    inv_freq = inv_freq_table(cfg, dtype)
    x = embedding(w["model.embed_tokens.weight"], tokens)
    for l in range(cfg["num_hidden_layers"]):
        x = layer(cfg, w, l, x, positions, inv_freq)
    x = rmsnorm(x, w["model.norm.weight"], float(cfg.get("rms_norm_eps", 1e-6)))
    head = w.get("lm_head.weight")
    if head is None:
        head = w["model.embed_tokens.weight"]
    return linear(x, head)


# ------------------------------------------------------------------- sampling
MASK64 = (1 << 64) - 1
GOLDEN = 0x9E3779B97F4A7C15


def splitmix64(z):
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
    return z ^ (z >> 31)


def mix_seed(seed, index):
    """Key of request `index`'s stream: splitmix64(seed + (index+1)*golden).  Not in the
    reference, whose generator is one global LCG stream (src/sampler.rs:3-12)."""
    return splitmix64((seed + (index + 1) * GOLDEN) & MASK64)


def uniform(key, n):
    """The n-th uniform of a stream: top 24 bits of splitmix64(key + (n+1)*golden), in
    [0, 1).  The reference draws (s >> 33) / u32::MAX from its LCG (src/sampler.rs:7-12),
    a 31-bit value over 2^32 that never exceeds one half; that is not restated."""
    return (splitmix64((key + (n + 1) * GOLDEN) & MASK64) >> 40) / 16777216.0


def greedy(logits):
    """Index of the largest logit (src/sampler.rs:15-19); of equal maxima the lowest
    index here (the reference's max_by keeps the last; ties do not occur in tests)."""
    return int(torch.argmax(logits))


def apply_rep_penalty(logits, recent, penalty):
    """Positive logits of recent tokens are divided by the penalty, others multiplied;
    once per occurrence in `recent` (src/sampler.rs:23-30)."""
    if penalty == 1.0:
        return logits
    logits = logits.clone()
    for t in recent:
        if 0 <= t < logits.numel():
            logits[t] = logits[t] / penalty if logits[t] > 0 else logits[t] * penalty
    return logits


def sample(logits, temperature, top_k, top_p, rep_penalty, recent, u):
    """The reference's sampler (src/sampler.rs:35-79) with the uniform `u` given:
    penalty; temperature <= 0 is greedy; logits / temperature; the top_k largest
    survive when 0 < top_k < V; softmax over them; top_p < 1 keeps the smallest
    prefix (in descending order) whose sum reaches top_p and renormalises; then the
    first token whose cumulative probability exceeds u, else the last survivor.
    The walk goes over the survivors in index order here (the reference walks them in
    descending order; the distribution is the same)."""
    logits = apply_rep_penalty(logits.to(torch.float32), recent, rep_penalty)
    if temperature <= 0.0:
        return greedy(logits)
    z = logits / temperature
    V = z.numel()
    order = sorted(range(V), key=lambda i: (-float(z[i]), i))
    if 0 < top_k < V:
        order = order[:top_k]
    zs = z[order]
    p = torch.exp(zs - zs[0])
    p = p / p.sum()
    if top_p < 1.0:
        cum, cut = 0.0, len(order)
        for i in range(len(order)):
            cum += float(p[i])
            if cum >= top_p:
                cut = i + 1
                break
        order, p = order[:cut], p[:cut]
        p = p / p.sum()
    keep = sorted(zip(order, p.tolist()))
    cum = 0.0
    for idx, pi in keep:
        cum += pi
        if u < cum:
            return idx
    return keep[-1][0]


def generate(cfg, w, prompt, max_tokens, temperature=0.0, top_k=0, top_p=1.0, rep_penalty=1.0,
             seed=0, index=0, stop=(), max_len=None, dtype=torch.float32):
    """One request, recomputing the whole sequence for every token, in the order of the
    reference's loop (src/main.rs:279-311): sample from the last logits; a stop token
    ends without being emitted; then the count limit; then the context limit
    (pos >= ctx - 1); emit, remember in the ring of 64, run the model on it."""
    seq, out, recent = list(prompt), [], []
    key = mix_seed(seed, index)
    ctx = max_len or cfg.get("max_position_embeddings", 32768)
    while True:
        logits = forward(cfg, w, seq, dtype)[-1]
        u = uniform(key, len(out))
        nxt = sample(logits, temperature, top_k, top_p, rep_penalty, recent, u)
        if nxt in stop or len(out) >= max_tokens or len(seq) >= ctx - 1:
            break
        out.append(nxt)
        recent.append(nxt)
        if len(recent) > 64:
            recent.pop(0)
        seq.append(nxt)
    return out


# -------------------------------------------------------------------- weights
def weight_shapes(cfg):
    """Tensor names and shapes of a Llama model folder, [out, in] matrices
    (src/model/llama.rs:122-143 with the safetensors names)."""
    E, F, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], kv_heads_of(cfg), head_dim_of(cfg)
    s = {"model.embed_tokens.weight": (V, E), "model.norm.weight": (E,)}
    if not cfg.get("tie_word_embeddings", False):
        s["lm_head.weight"] = (V, E)
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        s[p + "input_layernorm.weight"] = (E,)
        s[p + "post_attention_layernorm.weight"] = (E,)
        s[p + "self_attn.q_proj.weight"] = (nh * hd, E)
        s[p + "self_attn.k_proj.weight"] = (nkv * hd, E)
        s[p + "self_attn.v_proj.weight"] = (nkv * hd, E)
        s[p + "self_attn.o_proj.weight"] = (E, nh * hd)
        if cfg.get("attention_bias", False):
            s[p + "self_attn.q_proj.bias"] = (nh * hd,)
            s[p + "self_attn.k_proj.bias"] = (nkv * hd,)
            s[p + "self_attn.v_proj.bias"] = (nkv * hd,)
        s[p + "mlp.gate_proj.weight"] = (F, E)
        s[p + "mlp.up_proj.weight"] = (F, E)
        s[p + "mlp.down_proj.weight"] = (E, F)
    return s


def random_weights(cfg, seed, std=0.02, norm_noise=0.0, qk_std=None):
    """N(0, std) matrices, norm weights of one (+ noise when asked, so that a test sees
    a norm weight that is ignored), biases N(0, std).  qk_std: the deviation of the q and k
    matrices, for tests that need attention to be peaked (see tests/tiny.py)."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in weight_shapes(cfg).items():
        if name.endswith("norm.weight") or name.endswith("layernorm.weight"):
            w[name] = torch.ones(shape) + norm_noise * torch.randn(shape, generator=g)
        elif qk_std and (name.endswith("q_proj.weight") or name.endswith("k_proj.weight")):
            w[name] = torch.randn(shape, generator=g) * qk_std
        else:
            w[name] = torch.randn(shape, generator=g) * std
    return w

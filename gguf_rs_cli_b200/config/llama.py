"""Typed configuration of the Llama dense decoder, read from config.json's own keys.

What the reference reads from GGUF metadata (src/model/config.rs:20-47) maps to:
embedding_length -> hidden_size, block_count -> num_hidden_layers,
feed_forward_length -> intermediate_size, attention.head_count ->
num_attention_heads, attention.head_count_kv -> num_key_value_heads (default: the
head count, config.rs:35), context_length -> max_position_embeddings (default
32768, config.rs:41), rope.freq_base -> rope_theta (default 10000, config.rs:43),
attention.layer_norm_rms_epsilon -> rms_norm_eps (default 1e-6, config.rs:44).
head_dim defaults to hidden_size / heads (config.rs:48).  Required keys that are
missing raise an error naming the key, as config.rs:26 does.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .registry import ConfigError, register_architecture
from .specs import LayerSpec, ModelSpec, PartSpec, Run


@dataclass(frozen=True)
class RopeScaling:
    rope_type: str                      # "llama3" or "linear"
    factor: float
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 8192


def _need(raw: Dict[str, Any], key: str, kind=int):
    if key not in raw or raw[key] is None:
        raise ConfigError(f"config.json: missing key '{key}'")
    v = raw[key]
    if kind is int:
        if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
            raise ConfigError(f"config.json: '{key}' must be an integer, got {v!r}")
        return int(v)
    if kind is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json: '{key}' must be a number, got {v!r}")
        return float(v)
    return v


def _opt(raw, key, default, kind=int):
    if key not in raw or raw[key] is None:
        return default
    return _need(raw, key, kind)


def _head_dim_default(hidden: int, heads: int) -> int:
    """head_dim = hidden_size / heads when config.json gives none (src/model/config.rs:48); the division
    must come out even, else the projections' shapes would not match the folder's."""
    if hidden % heads:
        raise ConfigError(f"config.json: hidden_size {hidden} is not a multiple of num_attention_heads {heads} "
                          f"(and there is no 'head_dim')")
    return hidden // heads


def _id_list(v) -> List[int]:
    """An id or a list of ids (the reference takes eos ids as scalar or list,
    src/gguf/types.rs:24-29)."""
    if v is None:
        return []
    if isinstance(v, (list, tuple)):
        return [int(x) for x in v]
    return [int(v)]


@dataclass(frozen=True)
class LlamaConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int = 32768
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    rope_scaling: Optional[RopeScaling] = None
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    hidden_act: str = "silu"
    bos_token_id: Optional[int] = None
    eos_token_ids: List[int] = field(default_factory=list)
    torch_dtype: str = "bfloat16"

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "LlamaConfig":
        heads = _need(raw, "num_attention_heads")
        hidden = _need(raw, "hidden_size")
        if heads <= 0:
            raise ConfigError("config.json: 'num_attention_heads' must be positive")
        scaling = None
        rs = raw.get("rope_scaling")
        if rs:
            kind = rs.get("rope_type", rs.get("type"))
            if kind in ("llama3", "linear"):
                scaling = RopeScaling(
                    rope_type=kind,
                    factor=_need(rs, "factor", float),
                    low_freq_factor=_opt(rs, "low_freq_factor", 1.0, float),
                    high_freq_factor=_opt(rs, "high_freq_factor", 4.0, float),
                    original_max_position_embeddings=_opt(rs, "original_max_position_embeddings", 8192),
                )
            elif kind not in (None, "default"):
                raise ConfigError(f"config.json: rope_scaling type {kind!r} is not supported (llama3, linear, default)")
        cfg = cls(
            vocab_size=_need(raw, "vocab_size"),
            hidden_size=hidden,
            intermediate_size=_need(raw, "intermediate_size"),
            num_hidden_layers=_need(raw, "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=_opt(raw, "num_key_value_heads", heads),
            head_dim=(_need(raw, "head_dim") if raw.get("head_dim") is not None else _head_dim_default(hidden, heads)),
            max_position_embeddings=_opt(raw, "max_position_embeddings", 32768),
            rms_norm_eps=_opt(raw, "rms_norm_eps", 1e-6, float),
            rope_theta=_opt(raw, "rope_theta", 10000.0, float),
            rope_scaling=scaling,
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            attention_bias=bool(raw.get("attention_bias", False)),
            hidden_act=str(raw.get("hidden_act", "silu")),
            bos_token_id=raw.get("bos_token_id"),
            eos_token_ids=_id_list(raw.get("eos_token_id")),
            torch_dtype=str(raw.get("torch_dtype", raw.get("dtype", "bfloat16"))),
        )
        if raw.get("mlp_bias", False):
            raise ConfigError("config.json: 'mlp_bias' true is not supported (the feed-forward has no biases)")
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for k in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                  "num_attention_heads", "num_key_value_heads", "head_dim", "max_position_embeddings"):
            if getattr(self, k) <= 0:
                raise ConfigError(f"config.json: '{k}' must be positive, got {getattr(self, k)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(f"config.json: num_attention_heads {self.num_attention_heads} is not a multiple of "
                              f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"config.json: head_dim {self.head_dim} must be even (rotation pairs i with i+hd/2)")
        if self.hidden_act != "silu":
            raise ConfigError(f"config.json: hidden_act {self.hidden_act!r} is not supported (silu)")
        if not self.rms_norm_eps > 0:
            raise ConfigError("config.json: 'rms_norm_eps' must be positive")
        if self.rope_scaling and self.rope_scaling.factor <= 0:
            raise ConfigError("config.json: rope_scaling.factor must be positive")

    def to_dict(self) -> Dict[str, Any]:
        """config.json content that `from_dict` reads back to an equal configuration."""
        d: Dict[str, Any] = {
            "architectures": ["LlamaForCausalLM"], "model_type": "llama",
            "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size, "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads, "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim, "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps, "rope_theta": self.rope_theta, "rope_scaling": None,
            "tie_word_embeddings": self.tie_word_embeddings, "attention_bias": self.attention_bias,
            "mlp_bias": False, "hidden_act": self.hidden_act, "bos_token_id": self.bos_token_id,
            "eos_token_id": (self.eos_token_ids[0] if len(self.eos_token_ids) == 1 else (self.eos_token_ids or None)),
            "torch_dtype": self.torch_dtype,
        }
        if self.rope_scaling:
            s = self.rope_scaling
            d["rope_scaling"] = {"rope_type": s.rope_type, "factor": s.factor}
            if s.rope_type == "llama3":
                d["rope_scaling"].update(low_freq_factor=s.low_freq_factor, high_freq_factor=s.high_freq_factor,
                                         original_max_position_embeddings=s.original_max_position_embeddings)
        return d


def build_llama_spec(cfg: LlamaConfig) -> ModelSpec:
    """Llama as data: every layer is a pre-norm block of grouped-query attention with
    rotary positions and a gated SiLU feed-forward, run once each in order
    (src/model/llama.rs:361-404); tensor names follow src/model/llama.rs:122-143 in
    their safetensors spelling."""
    rope = PartSpec("rope", dict(
        head_dim=cfg.head_dim, rotary_dim=cfg.head_dim, theta=cfg.rope_theta, pairing="half",
        scaling=(None if cfg.rope_scaling is None else dict(
            rope_type=cfg.rope_scaling.rope_type, factor=cfg.rope_scaling.factor,
            low_freq_factor=cfg.rope_scaling.low_freq_factor, high_freq_factor=cfg.rope_scaling.high_freq_factor,
            original_max_position_embeddings=cfg.rope_scaling.original_max_position_embeddings))))
    layers = []
    for l in range(cfg.num_hidden_layers):
        p = f"model.layers.{l}."
        attn_tensors = {"q": p + "self_attn.q_proj.weight", "k": p + "self_attn.k_proj.weight",
                        "v": p + "self_attn.v_proj.weight", "o": p + "self_attn.o_proj.weight"}
        if cfg.attention_bias:
            attn_tensors.update({"q_bias": p + "self_attn.q_proj.bias", "k_bias": p + "self_attn.k_proj.bias",
                                 "v_bias": p + "self_attn.v_proj.bias"})
        layers.append(LayerSpec(
            block="prenorm",
            mixer=PartSpec("attention", dict(
                hidden_size=cfg.hidden_size, num_heads=cfg.num_attention_heads,
                num_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim,
                scale=cfg.head_dim ** -0.5, window=None, bias=cfg.attention_bias), attn_tensors),
            feed_forward=PartSpec("gated_mlp", dict(
                hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size, activation=cfg.hidden_act),
                {"gate": p + "mlp.gate_proj.weight", "up": p + "mlp.up_proj.weight",
                 "down": p + "mlp.down_proj.weight"}),
            norms={"mixer": PartSpec("rmsnorm", dict(size=cfg.hidden_size, eps=cfg.rms_norm_eps),
                                     {"weight": p + "input_layernorm.weight"}),
                   "feed_forward": PartSpec("rmsnorm", dict(size=cfg.hidden_size, eps=cfg.rms_norm_eps),
                                            {"weight": p + "post_attention_layernorm.weight"})},
            position=rope))
    # the head falls back to the embedding table whenever the folder has no matrix for it, whatever
    # tie_word_embeddings says (src/model/llama.rs:124); the flag only decides what random weights hold
    head_params = dict(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
                       tied_to="model.embed_tokens.weight", tied=cfg.tie_word_embeddings)
    spec = ModelSpec(
        architecture="LlamaForCausalLM",
        vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
        embedding=PartSpec("embedding", dict(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size),
                           {"weight": "model.embed_tokens.weight"}),
        layers=layers,
        schedule=[Run(l) for l in range(cfg.num_hidden_layers)],
        final_norm=PartSpec("rmsnorm", dict(size=cfg.hidden_size, eps=cfg.rms_norm_eps),
                            {"weight": "model.norm.weight"}),
        head=PartSpec("lm_head", head_params, {"weight": "lm_head.weight"}),
        max_position=cfg.max_position_embeddings,
        stop_token_ids=list(cfg.eos_token_ids),
        bos_token_id=cfg.bos_token_id,
        # older exports keep each layer's table of rotation frequencies beside the parameters
        ignored_tensors=["*.rotary_emb.inv_freq"],
    )
    spec.validate()
    return spec


register_architecture("LlamaForCausalLM", LlamaConfig, build_llama_spec, "llama")

import json

import pytest

from gguf_rs_cli_b200.config import (ConfigError, LlamaConfig, PartSpec, Run, load_config, registered_architectures)
from gguf_rs_cli_b200.config.specs import ModelSpec
from tests.tiny import config


def test_registry_names_llama():
    assert "LlamaForCausalLM" in registered_architectures() and "llama" in registered_architectures()


def test_typed_config_reads_every_key():
    arch, cfg = load_config(config("B"))
    assert isinstance(cfg, LlamaConfig) and arch.name == "LlamaForCausalLM"
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads) == (3, 96, 4, 1)
    assert (cfg.head_dim, cfg.intermediate_size, cfg.vocab_size) == (24, 224, 384)
    assert cfg.rope_theta == 500000.0 and cfg.rms_norm_eps == 1e-6 and cfg.tie_word_embeddings and cfg.attention_bias
    assert cfg.rope_scaling.rope_type == "llama3" and cfg.rope_scaling.factor == 8.0
    assert cfg.rope_scaling.original_max_position_embeddings == 64
    assert cfg.eos_token_ids == [3, 5]


def test_defaults_follow_the_reference():
    raw = {"architectures": ["LlamaForCausalLM"], "vocab_size": 100, "hidden_size": 48, "intermediate_size": 80,
           "num_hidden_layers": 1, "num_attention_heads": 4}
    _, cfg = load_config(raw)
    assert cfg.num_key_value_heads == 4 and cfg.head_dim == 12
    assert cfg.max_position_embeddings == 32768 and cfg.rope_theta == 10000.0 and cfg.rms_norm_eps == 1e-6
    assert cfg.rope_scaling is None and not cfg.tie_word_embeddings


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                                 "num_attention_heads"])
def test_missing_required_key_is_named(key):
    raw = config("A")
    del raw[key]
    with pytest.raises(ConfigError, match=key):
        load_config(raw)


def test_bad_values_are_refused():
    for key, val, pat in [("num_key_value_heads", 3, "multiple"), ("head_dim", 15, "even"),
                          ("hidden_act", "gelu", "hidden_act"), ("num_hidden_layers", 0, "positive"),
                          ("vocab_size", "many", "integer"), ("mlp_bias", True, "mlp_bias")]:
        raw = config("A")
        raw[key] = val
        with pytest.raises(ConfigError, match=pat):
            load_config(raw)
    raw = config("A")
    raw["rope_scaling"] = {"rope_type": "yarn", "factor": 2.0}
    with pytest.raises(ConfigError, match="yarn"):
        load_config(raw)


def test_unknown_architecture_lists_registered():
    with pytest.raises(ConfigError, match="LlamaForCausalLM"):
        load_config({"architectures": ["MambaForCausalLM"]})
    with pytest.raises(ConfigError, match="no architecture"):
        load_config({"vocab_size": 3})


def test_config_json_round_trip(tmp_path):
    _, cfg = load_config(config("B"))
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
    _, again = load_config(str(tmp_path))
    assert again == cfg
    with pytest.raises(ConfigError, match="no config.json"):
        load_config(str(tmp_path / "nowhere"))


def test_generation_config_adds_stop_tokens(tmp_path):
    raw = config("A")                                          # eos_token_id 2
    for extra, want in ((None, [2]), ({"eos_token_id": [2, 7, 9]}, [2, 7, 9]), ({"eos_token_id": 11}, [2, 11]), ({"top_p": 0.9}, [2])):
        d = tmp_path / f"m{want[-1]}{len(want)}{extra is None}"
        d.mkdir()
        (d / "config.json").write_text(json.dumps(raw))
        if extra is not None:
            (d / "generation_config.json").write_text(json.dumps(extra))
        arch, cfg = load_config(str(d))
        assert cfg.eos_token_ids == want and arch.build_spec(cfg).stop_token_ids == want
    (d / "generation_config.json").write_text("[1]")
    with pytest.raises(ConfigError, match="generation_config.json"):
        load_config(str(d))


def test_spec_is_data_layer_by_layer():
    arch, cfg = load_config(config("A"))
    spec = arch.build_spec(cfg)
    assert len(spec.layers) == 2 and [r.layer for r in spec.schedule] == [0, 1]
    l0 = spec.layers[0]
    assert l0.mixer.kind == "attention" and l0.feed_forward.kind == "gated_mlp" and l0.block == "prenorm"
    assert l0.mixer.params["num_kv_heads"] == 2 and l0.mixer.params["window"] is None
    assert l0.norms["mixer"].params["eps"] == 1e-5 and l0.position.params["theta"] == 10000.0
    assert l0.mixer.tensors["q"] == "model.layers.0.self_attn.q_proj.weight"
    # presence decides (src/model/llama.rs:124): the head of every Llama names its stand-in, and the flag
    # only says whether random weights hold a matrix for it
    assert spec.head.params["tied_to"] == "model.embed_tokens.weight" and spec.head.params["tied"] is False
    _, cfg_b = load_config(config("B"))
    assert arch.build_spec(cfg_b).head.params["tied"] is True
    assert spec.ignored_tensors == ["*.rotary_emb.inv_freq"]


def test_head_dim_must_divide_when_it_is_not_given():
    raw = config("A")
    del raw["head_dim"]
    assert load_config(raw)[1].head_dim == 16
    raw["num_attention_heads"], raw["num_key_value_heads"] = 6, 2
    with pytest.raises(ConfigError, match="not a multiple of num_attention_heads"):
        load_config(raw)
    raw["head_dim"] = 16                                      # given: any width goes
    assert load_config(raw)[1].head_dim == 16


def test_schedule_validation():
    arch, cfg = load_config(config("A"))
    spec = arch.build_spec(cfg)
    bad = ModelSpec(**{**spec.__dict__, "schedule": [Run(0), Run(5)]})
    with pytest.raises(ValueError, match="layer 5"):
        bad.validate()
    bad = ModelSpec(**{**spec.__dict__, "schedule": [Run(0), Run(1, cache_of=1)]})
    with pytest.raises(ValueError, match="earlier"):
        bad.validate()
    ok = ModelSpec(**{**spec.__dict__, "schedule": [Run(0), Run(1), Run(0)]})
    ok.validate()
    assert PartSpec("a", {"x": 1}).key() == PartSpec("a", {"x": 1}).key() != PartSpec("a", {"x": 2}).key()

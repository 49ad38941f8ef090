"""The tiny configurations the tests run: two Llama shapes that differ in every size
and option, as plain config.json dicts, plus helpers to make a model folder."""
import copy

TINY_A = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "intermediate_size": 176, "vocab_size": 256, "rope_theta": 10000.0, "rope_scaling": None,
    "rms_norm_eps": 1e-5, "max_position_embeddings": 128, "tie_word_embeddings": False,
    "hidden_act": "silu", "attention_bias": False, "eos_token_id": 2, "bos_token_id": 1,
}

TINY_B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 4, "num_key_value_heads": 1, "head_dim": 24,
    "intermediate_size": 224, "vocab_size": 384, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64},
    "rms_norm_eps": 1e-6, "max_position_embeddings": 256, "tie_word_embeddings": True,
    "hidden_act": "silu", "attention_bias": True, "eos_token_id": [3, 5], "bos_token_id": 0,
}

# A wider shape whose sizes reach the tensor-core and tiled kernels: head_dim 64, sizes
# that are multiples of 8 but of no power of two beyond that.
TINY_C = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 320, "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 64,
    "intermediate_size": 520, "vocab_size": 1000, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 128},
    "rms_norm_eps": 1e-5, "max_position_embeddings": 1024, "tie_word_embeddings": False,
    "hidden_act": "silu", "attention_bias": False, "eos_token_id": 2,
}

# Head size 128, wider than hidden / heads, so that a whole model reaches the tcgen05 attention kernel and the
# tensor-core products with a plain implementation beside it; an intermediate size that is no multiple of 64.
TINY_D = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 384, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 128,
    "intermediate_size": 360, "vocab_size": 520, "rope_theta": 10000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64},
    "rms_norm_eps": 3e-6, "max_position_embeddings": 512, "tie_word_embeddings": False,
    "hidden_act": "silu", "attention_bias": True, "eos_token_id": 7,
}

# Sizes that fit no fast kernel: a width and an intermediate size that are no multiples of 8 (the tensor-core
# product needs 16-byte rows), heads of 20, an odd vocabulary.  Whatever kernel runs, the result must be right.
TINY_E = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 100, "num_attention_heads": 5, "num_key_value_heads": 5, "head_dim": 20,
    "intermediate_size": 52, "vocab_size": 257, "rope_theta": 1000.0, "rope_scaling": None,
    "rms_norm_eps": 1e-5, "max_position_embeddings": 256, "tie_word_embeddings": True,
    "hidden_act": "silu", "attention_bias": False, "eos_token_id": 0,
}

CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E}


def qk_std(cfg, score_std=1.5):
    """Standard deviation of the q and k matrices under which attention scores have about `score_std`: with
    rows of unit RMS in front, a score q.k / sqrt(hd) has the deviation std^2 * hidden_size.  N(0, 0.02)
    everywhere gives scores of a few hundredths, attention that is nearly uniform, and a model whose logits
    hardly move when the rotation is wrong.  (Scores of deviation 3 and more make bfloat16's own rounding of q
    and k visible in the logits at the percent level: 1.5 keeps that noise inside the tests' tolerance while a
    missing rotation still moves the logits by 17 times the tolerance and more.)"""
    return (score_std / cfg["hidden_size"]) ** 0.5


def config(name):
    return copy.deepcopy(CONFIGS[name])

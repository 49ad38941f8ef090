"""A small, whole library for the Llama dense decoder on one NVIDIA B200: from a model
folder (config.json + safetensors) or random weights to generated token ids, on
hand-written sm_100a kernels.  config/, weights/, parts/, cache/, engine/ and sampling/ hold the
library, csrc/ the kernels, api.py and cli.py the two ways in."""
from .config import ConfigError, LlamaConfig, load_config, register_architecture, registered_architectures
from .sampling.params import SamplingParams

__all__ = ["ConfigError", "LlamaConfig", "load_config", "register_architecture", "registered_architectures",
           "SamplingParams", "LLM", "load", "from_random", "generate", "GenerationStats"]


def __getattr__(name):
    # the device-facing names import torch and the kernels only when asked for
    if name in ("LLM", "load", "from_random", "generate"):
        from . import api
        return getattr(api, name)
    if name == "GenerationStats":
        from .engine.generate import GenerationStats
        return GenerationStats
    raise AttributeError(name)

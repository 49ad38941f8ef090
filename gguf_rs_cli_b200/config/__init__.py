from .registry import (Architecture, ConfigError, load_config, read_config_json, register_architecture,
                       registered_architectures, resolve_architecture)
from .specs import LayerSpec, ModelSpec, PartSpec, Run
from .llama import LlamaConfig, RopeScaling, build_llama_spec

__all__ = ["Architecture", "ConfigError", "load_config", "read_config_json", "register_architecture",
           "registered_architectures", "resolve_architecture", "LayerSpec", "ModelSpec", "PartSpec", "Run",
           "LlamaConfig", "RopeScaling", "build_llama_spec"]

"""Random-weights mode: from a configuration and a seed to a model folder
(config.json, model.safetensors), or to tensors in memory for a model too large to
be worth writing.

What is written for a tensor is what the part that asks for it says (`TensorRequest.init`):
matrices and biases N(0, 0.02), norm weights ones.  Every tensor has its own generator,
seeded from (seed, tensor name), so a tensor's values do not depend on which other
tensors exist.  The reference has no such mode (it only reads GGUF
files, src/model/llama.rs:83-153).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Iterable, Tuple

import torch

from ..config.registry import load_config
from .loader import TensorRequest
from .safetensors_io import write_safetensors

STD = 0.02


def _seed_of(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def random_tensor(name: str, shape: Tuple[int, ...], seed: int, dtype=torch.bfloat16, device="cpu",
                  init: str = "normal") -> torch.Tensor:
    if init == "ones":
        return torch.ones(shape, dtype=dtype, device=device)
    if init == "zeros":
        return torch.zeros(shape, dtype=dtype, device=device)
    if init != "normal":
        raise ValueError(f"{name}: the random-weights mode knows no initial value {init!r} (normal, ones, zeros)")
    g = torch.Generator(device=device).manual_seed(_seed_of(seed, name))
    return (torch.randn(shape, generator=g, dtype=torch.float32, device=device) * STD).to(dtype)


def model_requests(raw_config: Dict) -> Iterable[TensorRequest]:
    """The tensors that the model of this configuration asks for."""
    from ..models.decoder import tensor_requests
    arch, cfg = load_config(raw_config)
    return tensor_requests(arch.build_spec(cfg))


def random_tensors(raw_config: Dict, seed: int, dtype=torch.bfloat16, device="cpu") -> Dict[str, torch.Tensor]:
    """name -> tensor for every tensor the model's parts want written (a tied head asks for
    none: its fallback stands in)."""
    out = {}
    for r in model_requests(raw_config):
        if r.init is None:
            continue
        if r.name not in out:
            out[r.name] = random_tensor(r.name, r.shape, seed, dtype, device, init=r.init)
    return out


def write_random_model(folder: str, raw_config: Dict, seed: int, dtype=torch.bfloat16) -> str:
    """Writes config.json and model.safetensors into `folder` and returns it."""
    os.makedirs(folder, exist_ok=True)
    tensors = random_tensors(raw_config, seed, dtype)
    cfg = dict(raw_config)
    cfg["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32", torch.float16: "float16"}[dtype]
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors.items(),
                      metadata={"format": "pt", "seed": seed})
    return folder

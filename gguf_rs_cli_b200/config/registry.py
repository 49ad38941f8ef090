"""The one registry from an architecture's name to its configuration class and its
model builder.  config.json's `architectures[0]` (or `model_type`) picks the entry.

The reference has no registry: one model struct serves every
`general.architecture` string and only prints it (src/main.rs:72-73,
src/model/config.rs:21-22).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict

from .specs import ModelSpec


class ConfigError(ValueError):
    """A config.json that cannot be used: missing key, bad value, unknown architecture."""


@dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: type
    build_spec: Callable[[Any], ModelSpec]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_cls: type, build_spec: Callable[[Any], ModelSpec], *aliases: str) -> None:
    """`config_cls.from_dict(dict)` must give the typed configuration and
    `build_spec(config)` the ModelSpec.  Aliases are `model_type` strings."""
    arch = Architecture(name, config_cls, build_spec)
    for n in (name,) + aliases:
        _ARCHITECTURES[n] = arch


def registered_architectures():
    return sorted(_ARCHITECTURES)


def resolve_architecture(raw: Dict[str, Any]) -> Architecture:
    names = list(raw.get("architectures") or [])
    if raw.get("model_type"):
        names.append(raw["model_type"])
    if not names:
        raise ConfigError("config.json names no architecture (keys 'architectures' or 'model_type')")
    for n in names:
        if n in _ARCHITECTURES:
            return _ARCHITECTURES[n]
    raise ConfigError(f"unsupported architecture {names}; registered: {registered_architectures()}")


def _eos_ids(value) -> list:
    return [] if value is None else [int(v) for v in value] if isinstance(value, (list, tuple)) else [int(value)]


def read_config_json(path: str) -> Dict[str, Any]:
    """config.json of a model folder (or the file itself).  A generation_config.json beside it adds its
    eos_token_id to the model's stop tokens, as the reference joins the tokenizer's end tokens with the
    chat template's (src/chat.rs:57-72)."""
    folder = path if os.path.isdir(path) else None
    raw = _read_json_object(os.path.join(path, "config.json") if folder else path)
    extra = os.path.join(folder, "generation_config.json") if folder else None
    if extra and os.path.exists(extra):
        more = _eos_ids(_read_json_object(extra).get("eos_token_id"))
        have = _eos_ids(raw.get("eos_token_id"))
        ids = have + [i for i in more if i not in have]
        if ids:
            raw["eos_token_id"] = ids[0] if len(ids) == 1 else ids
    return raw


def _read_json_object(path: str) -> Dict[str, Any]:
    try:
        with open(path, "r") as f:
            raw = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"no {os.path.basename(path) if path.endswith('.json') else 'config.json'} at {path}") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return raw


def load_config(path_or_dict):
    """Returns (architecture entry, typed configuration)."""
    raw = path_or_dict if isinstance(path_or_dict, dict) else read_config_json(path_or_dict)
    arch = resolve_architecture(raw)
    return arch, arch.config_cls.from_dict(raw)

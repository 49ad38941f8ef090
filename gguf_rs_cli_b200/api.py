"""The Python entry point: load a model folder (or make random weights), generate.

    from gguf_rs_cli_b200 import load, generate
    llm = load("/path/to/folder", dtype="bfloat16")
    ids = generate(llm, [[1, 2, 3], [4, 5]], max_tokens=16)

Token ids in, token ids out: the reference's tokenizer and chat templates
(src/tokenizer/) are not part of this library.
"""
from __future__ import annotations

import time
from typing import Callable, Dict, List, Optional, Sequence, Union

import torch

from .config.registry import load_config, read_config_json
from .engine.backend import EngineBackend
from .engine.generate import GenerationStats, generate_ids
from .engine.step import Engine
from .models.decoder import Decoder
from .sampling.params import SamplingParams
from .weights.loader import TensorSource, WeightStore
from .weights.random_init import random_tensors

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def _dtype(d) -> torch.dtype:
    if d not in _DTYPES:
        raise ValueError(f"dtype {d!r} is not supported (bfloat16 or float32)")
    return _DTYPES[d]


class LLM:
    """A loaded model and, once needed, an engine with a cache sized for the call."""

    def __init__(self, model: Decoder, raw_config: Dict):
        self.model, self.raw_config = model, raw_config
        self.spec = model.spec
        self._engine: Optional[Engine] = None
        self._engine_key = None
        self._backend: Optional[EngineBackend] = None

    def engine(self, n_tokens: int, n_slots: int, max_len: Optional[int] = None) -> Engine:
        """An engine whose cache has at least this room; the one at hand is kept when it
        is large enough and idle, else a new one replaces it."""
        key = (n_tokens, n_slots, max_len)
        e = self._engine
        if (e is not None and e.cache.slots.held_count == 0 and e.cache.n_slots >= n_slots
                and e.cache.n_pages * 64 >= n_tokens and e.cache.max_len >= (max_len or self.spec.max_position)):
            return e
        # too small, or still holding sequences that an interrupted caller left behind: a new one
        self._backend = None
        self._engine = None              # free the old cache before the new one is made
        self._engine = Engine(self.model, n_tokens=n_tokens, n_slots=n_slots, max_len=max_len)
        self._engine_key = key
        return self._engine

    def backend(self, n_tokens: int, n_slots: int, max_len: Optional[int] = None) -> EngineBackend:
        eng = self.engine(n_tokens, n_slots, max_len)
        if self._backend is None:
            self._backend = EngineBackend(eng)
        return self._backend


def _build(raw: Dict, source: TensorSource, dtype, device) -> LLM:
    arch, cfg = load_config(raw)
    dt = _dtype(dtype)
    model = Decoder(arch.build_spec(cfg), dt, torch.device(device))
    model.load(WeightStore(source, dt, torch.device(device)))
    return LLM(model, raw)


def load(path: str, dtype="bfloat16", device="cuda:0") -> LLM:
    """A folder with config.json and model.safetensors (or its shards).  The model class
    is chosen by config.json."""
    return _build(read_config_json(path), TensorSource.from_folder(path), dtype, device)


def from_random(config: Union[str, Dict], seed: int = 0, dtype="bfloat16", device="cuda:0") -> LLM:
    """Random weights N(0, 0.02) for a config.json (path or dict), made on `device` without
    touching the disk.  (`weights.write_random_model` writes the same kind of model as a
    folder.)"""
    raw = config if isinstance(config, dict) else read_config_json(config)
    tensors = random_tensors(raw, seed, dtype=_dtype(dtype), device=device)
    return _build(raw, TensorSource(tensors=tensors, where="random weights"), dtype, device)


def generate(llm: LLM, prompt_ids: Sequence[Sequence[int]], max_tokens: int = 512, temperature: float = 0.0,
             top_k: int = 0, top_p: float = 1.0, rep_penalty: float = 1.0, seed: int = 42,
             stop_token_ids: Optional[Sequence[int]] = None, max_batch: int = 64, ctx_len: Optional[int] = None,
             on_token: Optional[Callable[[int, int], None]] = None,
             stats: Optional[GenerationStats] = None, profile: bool = False) -> List[List[int]]:
    """Generated ids for each prompt, in order.  Option names and meanings are the
    reference's (src/main.rs:13-50): max_tokens, temperature (<= 0 is greedy), top_k,
    top_p, rep_penalty, seed, ctx_len (positions one sequence may hold).  Stop tokens
    default to the model's eos ids; a stop token ends a sequence and is not returned.
    profile: every step runs without CUDA graphs, with a time stamp after each stage, and prints
    one line to standard error (the reference's --debug-gpu, src/main.rs:45-47)."""
    prompts = [list(p) for p in prompt_ids]
    if not prompts:
        return []
    limit = min(ctx_len or llm.spec.max_position, llm.spec.max_position)
    batch = min(max_batch, len(prompts))
    longest = sorted((min(len(p) + max_tokens, limit) for p in prompts), reverse=True)[:batch]
    n_tokens = sum(((n + 63) // 64) * 64 for n in longest)
    backend = llm.backend(n_tokens=n_tokens, n_slots=batch, max_len=limit)
    stops = llm.spec.stop_token_ids if stop_token_ids is None else stop_token_ids
    params = SamplingParams(temperature, top_k, top_p, rep_penalty, seed)
    backend.profile = bool(profile)

    def clock():
        torch.cuda.synchronize()
        return time.perf_counter()

    return generate_ids(backend, prompts, max_tokens, params, stops, max_batch=batch, on_token=on_token, stats=stats,
                        clock=clock if stats is not None else None, context_limit=limit)

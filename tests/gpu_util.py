"""Helpers of the GPU tests: models with random weights both as an engine and as the
plain reference's dicts, and the comparison every test uses."""
import functools

import torch

from tests import plain_llama as P
from tests.tiny import config, qk_std

# Largest |engine - plain| allowed, relative to the largest |plain| of the compared block.
TOL = {"float32": 1e-4, "bfloat16": 2e-2}


def assert_close(got, want, dtype, what=""):
    got, want = got.detach().float().cpu(), want.detach().float().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} != {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    err = float((got - want).abs().max())
    ref = float(want.abs().max())
    assert err <= TOL[dtype] * max(ref, 1e-6), f"{what}: max error {err:.3e} against max |ref| {ref:.3e} ({dtype})"


@functools.lru_cache(maxsize=None)
def plain_weights(name, seed=0, norm_noise=0.1):
    """Weights on the CPU, rounded to bfloat16 values so that both dtypes of the engine
    hold exactly the same numbers as the plain reference.  q and k are scaled so that attention is
    peaked: a wrong rotation, a dropped frequency scaling or a wrong head group then moves the logits by
    many times the bfloat16 tolerance (tests/test_plain.py shows it)."""
    w = P.random_weights(config(name), seed, norm_noise=norm_noise, qk_std=qk_std(config(name)))
    return {k: v.to(torch.bfloat16).to(torch.float32) for k, v in w.items()}


@functools.lru_cache(maxsize=None)
def llm(name, dtype, seed=0):
    from gguf_rs_cli_b200.api import _build
    from gguf_rs_cli_b200.weights import TensorSource
    w = {k: v.to(torch.bfloat16) for k, v in plain_weights(name, seed).items()}
    return _build(config(name), TensorSource(tensors=w, where=f"tiny {name}"), dtype, "cuda:0")


def new_engine(name, dtype, n_tokens=1024, n_slots=8, **kw):
    from gguf_rs_cli_b200.engine.step import Engine
    return Engine(llm(name, dtype).model, n_tokens=n_tokens, n_slots=n_slots, **kw)


def tokens_of(name, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, config(name)["vocab_size"], (n,), generator=g).tolist()


@functools.lru_cache(maxsize=None)
def plain_logits(name, n, seed):
    return P.forward(config(name), plain_weights(name), tokens_of(name, n, seed))

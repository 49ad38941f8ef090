#!/usr/bin/env python3
"""Makes the golden logits under tests/golden/ with the C++ restatement of the reference's CPU forward pass.

The reference itself (Smoffyy/gguf-rs-cli) is a Rust program with a Vulkan path; neither can be compiled,
imported or run where this library is built (no cargo, rustc or graphics stack, no network).  So the golden
numbers do not come from a run of the reference: they come from baseline/cpu_ref.cpp, a plain C++ program
written from the same lines of the reference as tests/plain_llama.py (src/model/llama.rs:343-409,
src/math/ops.rs, src/math/rope.rs) but independently of it: token by token with a cache, scalar loops, its own
safetensors and config readers.  tests/test_golden.py checks the plain implementation (whole sequences, torch)
against these files, so that a misreading would have to be made twice, in two languages, to go unseen.

    python tests/golden/make_golden.py        # rewrites tests/golden/tiny_{A,B,D}.json

Each file holds the token ids, a fingerprint of the seeded weights (so that a change of the generator shows as
such), and the logits of every position rounded to 9 significant digits.
"""
import json
import os
import subprocess
import sys
import tempfile

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from tests import plain_llama as P                      # noqa: E402
from tests.tiny import config, qk_std                   # noqa: E402

CASES = {"A": (11, 14), "B": (12, 18), "D": (13, 9)}    # name -> (weights seed, number of tokens)


def build_cpu_ref(folder):
    exe = os.path.join(folder, "cpu_ref")
    subprocess.run(["g++", "-O2", "-fopenmp", "-std=c++17", os.path.join(ROOT, "baseline", "cpu_ref.cpp"), "-o", exe], check=True)
    return exe


def case_inputs(name):
    """Seeded weights (rounded to bfloat16 values, q and k scaled so that attention is peaked) and tokens."""
    seed, n = CASES[name]
    cfg = config(name)
    w = P.random_weights(cfg, seed, norm_noise=0.1, qk_std=qk_std(cfg))
    w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    g = torch.Generator().manual_seed(seed + 100)
    tokens = torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist()
    fingerprint = float(sum(float(v.double().abs().sum()) for v in w.values()))
    return cfg, w, tokens, fingerprint


def run_cpu_ref(exe, cfg, w, tokens, folder):
    from gguf_rs_cli_b200.weights import write_safetensors
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), list(w.items()))          # 32-bit: exactly these values
    out = os.path.join(folder, "logits.f32")
    subprocess.run([exe, "--model", folder, "--tokens", ",".join(map(str, tokens)), "--out", out], check=True,
                   stdout=subprocess.DEVNULL)
    import numpy as np
    return torch.from_numpy(np.fromfile(out, dtype="<f4").reshape(len(tokens), cfg["vocab_size"]).copy())


def main():
    with tempfile.TemporaryDirectory() as tmp:
        exe = build_cpu_ref(tmp)
        for name in CASES:
            cfg, w, tokens, fingerprint = case_inputs(name)
            logits = run_cpu_ref(exe, cfg, w, tokens, os.path.join(tmp, name))
            path = os.path.join(ROOT, "tests", "golden", f"tiny_{name}.json")
            with open(path, "w") as f:
                json.dump({"made_by": "baseline/cpu_ref.cpp through tests/golden/make_golden.py", "config": name,
                           "tokens": tokens, "weights_fingerprint": fingerprint,
                           "logits": [[float(f"{x:.9g}") for x in row] for row in logits.tolist()]}, f)
            print(f"wrote {path}: {len(tokens)} x {cfg['vocab_size']} logits, largest {float(logits.abs().max()):.4f}")


if __name__ == "__main__":
    main()

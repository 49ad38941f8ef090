"""The plain implementation against a second, independent one: the committed golden logits were made by the C++
restatement of the reference's CPU forward pass (baseline/cpu_ref.cpp, token by token with a cache), and the
program itself is built and run here as well when a compiler is at hand."""
import json
import os
import shutil
import subprocess

import pytest
import torch

from tests import plain_llama as P
from tests.golden import make_golden as G

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("name", sorted(G.CASES))
def test_plain_implementation_equals_the_committed_golden_logits(name):
    with open(os.path.join(HERE, "golden", f"tiny_{name}.json")) as f:
        gold = json.load(f)
    cfg, w, tokens, fingerprint = G.case_inputs(name)
    assert tokens == gold["tokens"]
    assert abs(fingerprint - gold["weights_fingerprint"]) <= 1e-9 * fingerprint, "the seeded weights are not those of the golden file"
    want = torch.tensor(gold["logits"])
    got = P.forward(cfg, w, tokens)
    assert got.shape == want.shape
    ref = float(want.abs().max())
    assert float((got - want).abs().max()) <= 2e-5 * ref
    # and in 64-bit the plain implementation is closer still: both are sums of the same terms
    got64 = P.forward(cfg, w, tokens, torch.float64)
    assert float((got64 - want.double()).abs().max()) <= 2e-5 * ref


@pytest.mark.skipif(shutil.which("g++") is None, reason="no C++ compiler")
def test_cpu_reference_program_builds_and_agrees(tmp_path):
    exe = G.build_cpu_ref(str(tmp_path))
    cfg, w, tokens, _ = G.case_inputs("B")
    logits = G.run_cpu_ref(exe, cfg, w, tokens, str(tmp_path / "B"))
    want = P.forward(cfg, w, tokens)
    assert float((logits - want).abs().max()) <= 2e-5 * float(want.abs().max())
    # it refuses what it cannot run, in words
    r = subprocess.run([exe, "--model", str(tmp_path / "B"), "--tokens", "999999"], capture_output=True, text=True)
    assert r.returncode != 0 and "outside the vocabulary" in r.stderr
    r = subprocess.run([exe, "--model", str(tmp_path / "nowhere"), "--tokens", "1"], capture_output=True, text=True)
    assert r.returncode != 0 and "cannot open" in r.stderr

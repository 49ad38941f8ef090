import json
import os
import subprocess
import sys

import pytest
import torch

from gguf_rs_cli_b200.cli import build_parser, parse_ids
from tests.tiny import config

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_option_names_and_defaults_are_the_reference_s():
    a = build_parser().parse_args(["-m", "folder", "-p", "1,2,3"])
    assert (a.max_tokens, a.temperature, a.top_k, a.top_p, a.rep_penalty, a.ctx_len, a.seed) == (512, 0.7, 40, 0.9, 1.1, 8192, 42)
    assert not a.stats and not a.gpu and a.prompts == [[1, 2, 3]]
    a = build_parser().parse_args(["--model", "f", "--prompt-ids", "4 5", "-p", "6", "-n", "3", "-t", "0", "--top-k", "0", "--top-p",
                                   "1", "--rep-penalty", "1", "-c", "100", "--seed", "7", "--stats", "--gpu", "--debug-gpu"])
    assert a.prompts == [[4, 5], [6]] and (a.max_tokens, a.temperature, a.ctx_len, a.seed) == (3, 0.0, 100, 7) and a.stats
    assert parse_ids("1, 2,3") == [1, 2, 3]
    assert a.stop_ids is None and not a.no_eos and a.debug_gpu      # the model's own end tokens
    assert build_parser().parse_args(["-m", "f", "-p", "1", "--stop-ids", ""]).stop_ids == []
    b = build_parser().parse_args(["-m", "f", "-p", "1", "--stop-ids", "2,7", "--no-eos", "--profile"])
    assert b.stop_ids == [2, 7] and b.no_eos and b.debug_gpu
    with pytest.raises(SystemExit):
        build_parser().parse_args(["-p", "1"])                     # no model
    with pytest.raises(SystemExit):
        build_parser().parse_args(["-m", "f", "-p", "one"])


@pytest.mark.gpu
def test_cli_generates_what_the_entry_point_generates(tmp_path):
    from gguf_rs_cli_b200.api import generate, load
    from gguf_rs_cli_b200.weights import write_random_model
    folder = write_random_model(str(tmp_path / "m"), config("B"), seed=1, dtype=torch.bfloat16)
    prompts = [[5, 6, 7], [300, 2, 9, 11, 80]]
    args = ["-n", "6", "-t", "0.9", "--seed", "5", "--dtype", "float32", "--stop-ids", "383", "--no-eos", "--stats", "--debug-gpu"]
    cmd = [sys.executable, os.path.join(ROOT, "bin", "gguf-rs-cli"), "-m", folder] + args
    for p in prompts:
        cmd += ["-p", ",".join(map(str, p))]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    got = [[int(t) for t in line.split(",")] for line in r.stdout.strip().splitlines()]
    want = generate(load(folder, "float32"), prompts, max_tokens=6, temperature=0.9, top_k=40, top_p=0.9, rep_penalty=1.1, seed=5,
                    stop_token_ids=[383])
    assert got == want and all(len(g) == 6 for g in got)
    assert "[Stats] prefill: 8 tok in" in r.stderr and "generated: 12 tok" in r.stderr and "[GPU]" in r.stderr
    assert "EOS tokens: [383]" in r.stderr
    # --debug-gpu: one line per step with a stamp after every stage, as the reference prints its timestamps
    lines = [l for l in r.stderr.splitlines() if l.startswith("[GPU step")]
    assert len(lines) == 7 and lines[0].startswith("[GPU step of 8 tokens]") and lines[1].startswith("[GPU step of 2 tokens]")
    for stage in ("embed", "norm", "qkv", "attention", "o", "ff_norm", "gate_up", "down", "layers", "head", "sample", "total GPU"):
        assert f"[{stage}: " in lines[1], (stage, lines[1])
    # without --no-eos the model's end tokens (3 and 5 here) are joined with --stop-ids
    r2 = subprocess.run([a for a in cmd if a != "--no-eos"], capture_output=True, text=True)
    assert r2.returncode == 0 and "EOS tokens: [3, 5, 383]" in r2.stderr
    # a config for random weights, and a loud error for a broken folder
    cfg_path = tmp_path / "c.json"
    cfg_path.write_text(json.dumps(config("A")))
    r = subprocess.run([sys.executable, "-m", "gguf_rs_cli_b200", "--random", str(cfg_path), "-p", "1,2", "-n", "2", "-t", "0"],
                       capture_output=True, text=True, cwd=ROOT)
    assert r.returncode == 0 and len(r.stdout.strip().split(",")) == 2, r.stderr
    os.remove(os.path.join(folder, "model.safetensors"))
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 1 and "model.safetensors" in r.stderr


@pytest.mark.gpu
def test_kernel_stamps_program_reports_every_kernel_of_a_layer():
    """bin/kernel_stamps builds the library's second variant (time stamps inside the kernels) and reports, for
    the five kernels of a layer, where their CTAs pass the stamped places: every CTA enters, waits, and exits in
    that order, and the products that share tiles show the places of the sharing."""
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "kernel_stamps"), "--tokens", "8", "--layers", "2"],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    out = r.stdout
    for name in ("q/k/v product", "o product", "gate+up product", "down product", "decode attention"):
        assert f"--- {name}" in out
    blocks = out.split("--- ")[1:]
    assert "296 CTAs" in blocks[0] and "224 CTAs" in blocks[2] and "64 CTAs" in blocks[4]
    assert "partial sums stored and fenced" in blocks[0] and "partial sums stored and fenced" not in blocks[2]
    for b in blocks:
        med = {}
        for line in b.splitlines():
            if " median " in line and line.startswith("  ") and "per CTA" not in line:
                place = line[2:36].strip()
                med[place] = float(line.split("median")[1].split()[0])
        assert med["entry"] <= med["wait for the kernel in front over"] <= med["exit" if "exit" in med else "output written"]

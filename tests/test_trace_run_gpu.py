"""bin/trace_run as a user runs it: a model folder, steps on standard input, logits in files."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests import plain_llama as P
from tests.gpu_util import TOL
from tests.tiny import config, qk_std

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class Replay:
    def __init__(self, folder, dtype, out, max_tokens):
        self.out = out
        self.proc = subprocess.Popen([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                                      "--out", out, "--max-tokens", str(max_tokens)],
                                     stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
        self.n = 0

    def step(self, entries, end=()):
        rec = {"step": self.n, "entries": [{"id": i, "tokens": t, "want": list(w)} for i, t, w in entries], "end": list(end)}
        self.proc.stdin.write(json.dumps(rec) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline().strip()
        assert line == f"done {self.n}", f"trace_run said {line!r}"
        path = os.path.join(self.out, f"{self.n}.f32")
        self.n += 1
        if any(w for _, _, w in entries):
            return np.fromfile(path, dtype="<f4")
        assert not os.path.exists(path)
        return None

    def finish(self):
        self.proc.stdin.close()
        assert self.proc.wait(timeout=60) == 0


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    """Model folders in a temporary place: A as the random-weights mode writes it, B and D with q and k scaled
    so that attention is peaked (see tests/tiny.py), written by the package's own writer."""
    from gguf_rs_cli_b200.weights import TensorSource, write_random_model, write_safetensors
    out = {}
    for name in ("A", "B", "D"):
        folder = str(tmp_path_factory.mktemp(f"model{name}"))
        if name == "A":
            write_random_model(folder, config(name), seed=3, dtype=torch.bfloat16)
        else:
            w = P.random_weights(config(name), 3, norm_noise=0.1, qk_std=qk_std(config(name)))
            with open(os.path.join(folder, "config.json"), "w") as f:
                json.dump(config(name), f)
            write_safetensors(os.path.join(folder, "model.safetensors"), [(n, t.to(torch.bfloat16)) for n, t in w.items()])
        src = TensorSource.from_folder(folder)
        out[name] = (folder, {n: src.get(n).float() for n in src.names()})
    return out


def close(got, want, dtype, what):
    want = want.numpy().reshape(-1)
    assert got.shape == want.shape, f"{what}: {got.shape} values, expected {want.shape}"
    err, ref = float(np.abs(got - want).max()), float(np.abs(want).max())
    assert err <= TOL[dtype] * ref, f"{what}: max error {err:.3e} against {ref:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_replay_whole_one_by_one_and_unequal_batches(name, dtype, folders, tmp_path):
    folder, w = folders[name]
    cfg = config(name)
    g = torch.Generator().manual_seed(11)
    V = cfg["vocab_size"]
    seqs = {rid: torch.randint(0, V, (n,), generator=g).tolist() for rid, n in
            [("a", 100), ("b", 70), ("c", 5), ("d", 64), ("e", 33), ("f", 129), ("g", 1)]}
    want = {rid: P.forward(cfg, w, s) for rid, s in seqs.items()}
    # live at once at most: batch {a,b,c,d} = 128+128+64+64 = 384, then {e,f,g} = 64+192+64
    r = Replay(folder, dtype, str(tmp_path / "out"), max_tokens=384)
    # 1. a request alone and whole
    got = r.step([("a", seqs["a"], range(100))], end=["a"])
    close(got, want["a"], dtype, "whole")
    # 2. the same with the last 32 tokens one by one
    got = r.step([("a", seqs["a"][:68], range(68))])
    close(got, want["a"][:68], dtype, "prefix")
    for i in range(68, 100):
        got = r.step([("a", [seqs["a"][i]], [0])], end=["a"] if i == 99 else [])
        close(got, want["a"][i], dtype, f"position {i} decoded alone")
    # 3. batches of unequal lengths, shorter requests ending earlier, one batch after another
    for batch, decode in ((["a", "b", "c", "d"], 7), (["e", "f", "g"], 5)):
        n0 = {rid: len(seqs[rid]) - (decode - k) for k, rid in enumerate(batch)}     # later ones keep fewer for decoding
        n0 = {rid: max(1, min(n, len(seqs[rid]))) for rid, n in n0.items()}
        got = r.step([(rid, seqs[rid][:n0[rid]], [n0[rid] - 1]) for rid in batch],
                     end=[rid for rid in batch if n0[rid] == len(seqs[rid])])
        close(got, torch.stack([want[rid][n0[rid] - 1] for rid in batch]), dtype, f"prompts of batch {batch}")
        fed = dict(n0)
        live = [rid for rid in batch if fed[rid] < len(seqs[rid])]
        while live:
            done = [rid for rid in live if fed[rid] + 1 == len(seqs[rid])]
            got = r.step([(rid, [seqs[rid][fed[rid]]], [0]) for rid in live], end=done)
            close(got, torch.stack([want[rid][fed[rid]] for rid in live]), dtype, f"decode step of {live}")
            for rid in live:
                fed[rid] += 1
            live = [rid for rid in live if rid not in done]
    # nothing wanted writes no file; an empty want list among others is skipped
    assert r.step([("h", seqs["c"], [])]) is None
    got = r.step([("h", [7], []), ("i", seqs["c"], [4])], end=["h", "i"])
    close(got, want["c"][4], dtype, "a request that wants nothing beside one that does")
    r.finish()


def test_replay_refuses_more_than_the_cache_holds(folders, tmp_path):
    folder, _ = folders["A"]
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                        "--out", str(tmp_path / "o"), "--max-tokens", "64"],
                       input=json.dumps({"step": 0, "entries": [{"id": "x", "tokens": [1] * 65, "want": [0]}], "end": []}) + "\n",
                       capture_output=True, text=True)
    assert p.returncode != 0 and "CacheFull" in p.stderr

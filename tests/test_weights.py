import json
import struct

import pytest
import torch

from gguf_rs_cli_b200.config import load_config
from gguf_rs_cli_b200.models import tensor_requests
from gguf_rs_cli_b200.weights import (SafetensorsFile, TensorSource, WeightError, WeightFileError, WeightStore,
                                      random_tensors, storage_dtype, write_random_model, write_safetensors)
from tests import plain_llama
from tests.tiny import config


def requests_of(raw):
    arch, cfg = load_config(raw)
    return tensor_requests(arch.build_spec(cfg))


def test_safetensors_round_trip(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int64).reshape(2, 3),
         "d": torch.randn(2, 2).to(torch.float16)}
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, t.items())
    f = SafetensorsFile(path)
    assert sorted(f.names()) == ["a", "b", "c", "d"]
    for n, v in t.items():
        assert f.shape(n) == tuple(v.shape) and f.dtype(n) == v.dtype
        assert torch.equal(f.tensor(n), v)
    # the installed safetensors package reads the same bytes
    from safetensors.torch import load_file
    for n, v in load_file(path).items():
        assert torch.equal(v, t[n])


def test_safetensors_rejects_broken_files(tmp_path):
    p = tmp_path / "short.safetensors"
    p.write_bytes(b"abc")
    with pytest.raises(WeightFileError, match="too short"):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(WeightFileError, match="header length"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4, 4], "data_offsets": [0, 64]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 32)          # data cut short
    with pytest.raises(WeightFileError, match="offsets"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"w": {"dtype": "Q4_0", "shape": [4], "data_offsets": [0, 4]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 4)
    with pytest.raises(WeightFileError, match="dtype"):
        SafetensorsFile(str(p))


def test_safetensors_header_escapes_metadata_and_unknown_keys(tmp_path):
    """The header is JSON: names may hold escapes, entries may hold keys this reader does not know, and
    __metadata__ is kept; a name listed twice and text after the header's end are refused."""
    p = tmp_path / "h.safetensors"
    data = torch.arange(6, dtype=torch.float32)
    raw = data.numpy().tobytes()
    hdr = ('{"__metadata__": {"format": "pt", "note": "a \\"quoted\\" \\u00e9\\ud83d\\ude00", "n": 3},'
           ' "layer\\u002e0/w\\t": {"dtype": "F32", "extra": [1, {"x": null}, "s"], "shape": [2, 3], "data_offsets": [0, 24]},'
           ' "empty": {"dtype": "BF16", "shape": [0, 4], "data_offsets": [24, 24]}}').encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + raw)
    f = SafetensorsFile(str(p))
    assert f.metadata == {"format": "pt", "note": 'a "quoted" \u00e9\U0001F600'}
    assert sorted(f.names()) == ["empty", "layer.0/w\t"]
    assert torch.equal(f.tensor("layer.0/w\t"), data.reshape(2, 3)) and f.tensor("empty").shape == (0, 4)
    view = f.tensor("layer.0/w\t")[1]
    del f                                                    # the map stays while a tensor views it
    assert view.tolist() == [3.0, 4.0, 5.0]
    twice = b'{"w": {"dtype": "U8", "shape": [1], "data_offsets": [0, 1]}, "w": {"dtype": "U8", "shape": [1], "data_offsets": [0, 1]}}'
    p.write_bytes(struct.pack("<Q", len(twice)) + twice + b"\0")
    with pytest.raises(WeightFileError, match="listed twice"):
        SafetensorsFile(str(p))
    for bad in (b'{"w": {"dtype": "U8", "shape": [1], "data_offsets": [0, 1]}} x', b'{"w": {"dtype": "U8", "shape": [1.5]}}', b'["w"]'):
        p.write_bytes(struct.pack("<Q", len(bad)) + bad + b"\0")
        with pytest.raises(WeightFileError, match="not JSON"):
            SafetensorsFile(str(p))
    with pytest.raises(WeightFileError, match="cannot open"):
        SafetensorsFile(str(tmp_path / "absent.safetensors"))


def test_names_and_shapes_match_the_plain_reference():
    for name in "AB":
        raw = config(name)
        want = plain_llama.weight_shapes(raw)
        got = {r.name: tuple(r.shape) for r in requests_of(raw) if r.init is not None}       # what random weights hold
        assert got == {k: tuple(v) for k, v in want.items()}
        inits = {r.name: r.init for r in requests_of(raw)}
        assert all((init == "ones") == (name.endswith("norm.weight")) for name, init in inits.items() if init)


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    raw = config("A")
    w = plain_llama.random_weights(raw, 0)
    del w["model.layers.1.mlp.up_proj.weight"]
    del w["model.norm.weight"]
    w["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(64, 64)
    w["model.layers.7.extra.weight"] = torch.zeros(2)
    store = WeightStore(TensorSource(tensors=w, where="test"), torch.float32, "cpu")
    with pytest.raises(WeightError) as e:
        store.check(requests_of(raw))
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.7.extra.weight"]
    assert err.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (32, 64), (64, 64))]
    text = str(err)
    for needle in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "expected [32, 64], found [64, 64]"):
        assert needle in text


def test_tied_head_falls_back_to_the_embedding():
    raw = config("B")
    w = plain_llama.random_weights(raw, 0)
    assert "lm_head.weight" not in w
    store = WeightStore(TensorSource(tensors=w), torch.float32, "cpu")
    reqs = requests_of(raw)
    store.check(reqs)
    head = [r for r in reqs if r.name == "lm_head.weight"][0]
    emb = [r for r in reqs if r.name == "model.embed_tokens.weight"][0]
    assert store.get(head) is store.get(emb)
    # presence decides, as in the reference (src/model/llama.rs:124): an untied configuration whose folder
    # has no head matrix uses the embedding too, and a tied one whose folder has a matrix uses that
    raw["tie_word_embeddings"] = False
    WeightStore(TensorSource(tensors=w), torch.float32, "cpu").check(requests_of(raw))
    assert "lm_head.weight" in random_tensors(raw, 0) and "lm_head.weight" not in random_tensors(config("B"), 0)
    w["lm_head.weight"] = torch.zeros(384, 96)
    store = WeightStore(TensorSource(tensors=w), torch.float32, "cpu")
    store.check(requests_of(config("B")))
    assert store.get(head) is not store.get(emb)


def test_buffers_of_older_exports_are_ignored_other_extras_are_not():
    raw = config("A")
    w = plain_llama.random_weights(raw, 0)
    w["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    arch, cfg = load_config(raw)
    spec = arch.build_spec(cfg)
    store = WeightStore(TensorSource(tensors=w, where="test"), torch.float32, "cpu")
    store.check(tensor_requests(spec), allow_unused=spec.ignored_tensors)
    with pytest.raises(WeightError, match="rotary_emb.inv_freq"):
        store.check(tensor_requests(spec))
    w["model.layers.0.self_attn.rotary_emb.other"] = torch.zeros(8)
    with pytest.raises(WeightError, match="rotary_emb.other"):
        WeightStore(TensorSource(tensors=w), torch.float32, "cpu").check(tensor_requests(spec), allow_unused=spec.ignored_tensors)


def write_shards(folder, tensors, split_at, twice=()):
    """model.safetensors.index.json and two shards; names in `twice` are stored in both."""
    names = sorted(tensors)
    a, b = names[:split_at], names[split_at:]
    files = {"model-00001-of-00002.safetensors": a + [n for n in twice if n not in a],
             "model-00002-of-00002.safetensors": b + [n for n in twice if n not in b]}
    weight_map = {}
    for fname, ns in files.items():
        write_safetensors(str(folder / fname), [(n, tensors[n]) for n in ns])
        for n in ns:
            weight_map[n] = fname
    (folder / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": weight_map}))


def test_sharded_folder(tmp_path):
    raw = config("A")
    w = {k: v.to(torch.bfloat16) for k, v in plain_llama.random_weights(raw, 2).items()}
    d = tmp_path / "sharded"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(raw))
    write_shards(d, w, split_at=7)
    src = TensorSource.from_folder(str(d))
    assert sorted(src.names()) == sorted(w)
    WeightStore(src, torch.bfloat16, "cpu").check(requests_of(raw))
    for n in ("model.embed_tokens.weight", "model.layers.1.mlp.down_proj.weight", "lm_head.weight"):       # from both shards
        assert torch.equal(src.get(n), w[n])
    # a tensor stored in both shards is named in the one error
    d2 = tmp_path / "twice"
    d2.mkdir()
    write_shards(d2, w, split_at=7, twice=["model.norm.weight"])
    with pytest.raises(WeightError, match=r"model.norm.weight \(stored in more than one shard\)"):
        TensorSource.from_folder(str(d2))
    # an index that names a shard that is not there
    d3 = tmp_path / "lost"
    d3.mkdir()
    write_shards(d3, w, split_at=7)
    (d3 / "model-00002-of-00002.safetensors").unlink()
    with pytest.raises(WeightFileError):
        TensorSource.from_folder(str(d3))


def test_file_written_by_the_installed_package_is_read_by_the_native_reader(tmp_path):
    from safetensors.torch import save_file
    t = {"w": torch.randn(5, 8).to(torch.bfloat16), "f": torch.randn(3), "h": torch.randn(4, 2).to(torch.float16),
         "i": torch.arange(10, dtype=torch.int64)}
    path = str(tmp_path / "pkg.safetensors")
    save_file(t, path, metadata={"format": "pt"})
    f = SafetensorsFile(path)
    assert sorted(f.names()) == sorted(t)
    for n, v in t.items():
        assert f.shape(n) == tuple(v.shape) and f.dtype(n) == v.dtype and torch.equal(f.tensor(n), v)


def test_storage_dtypes():
    bf, f32 = torch.bfloat16, torch.float32
    assert storage_dtype(torch.bfloat16, bf) == bf and storage_dtype(torch.float16, bf) == bf
    assert storage_dtype(torch.float32, bf) == f32            # stored in 32-bit stays so
    assert storage_dtype(torch.bfloat16, f32) == f32 and storage_dtype(torch.float32, f32) == f32
    assert storage_dtype(torch.int64, bf) == torch.int32
    w = {"a": torch.randn(4).to(torch.bfloat16), "n": torch.ones(4), "i": torch.arange(4)}
    s = WeightStore(TensorSource(tensors=w), bf, "cpu")
    from gguf_rs_cli_b200.weights import TensorRequest
    assert s.get(TensorRequest("a", (4,))).dtype == bf and s.get(TensorRequest("n", (4,))).dtype == f32
    assert s.get(TensorRequest("i", (4,))).dtype == torch.int32
    assert s.get(TensorRequest("zz", (4,), optional=True)) is None


def test_random_model_folder(tmp_path):
    raw = config("B")
    folder = write_random_model(str(tmp_path / "m"), raw, seed=5, dtype=torch.bfloat16)
    _, cfg = load_config(folder)
    assert cfg.hidden_size == 96 and cfg.torch_dtype == "bfloat16"
    src = TensorSource.from_folder(folder)
    WeightStore(src, torch.bfloat16, "cpu").check(requests_of(raw))
    again = random_tensors(raw, 5)
    other = random_tensors(raw, 6)
    n = "model.layers.2.mlp.down_proj.weight"
    assert torch.equal(src.get(n), again[n]) and not torch.equal(again[n], other[n])
    assert abs(float(again[n].float().std()) - 0.02) < 0.002
    assert torch.equal(again["model.norm.weight"].float(), torch.ones(96))
    # a tensor's values do not depend on which other tensors exist
    raw2 = config("B")
    raw2["num_hidden_layers"] = 4
    assert torch.equal(random_tensors(raw2, 5)[n], again[n])

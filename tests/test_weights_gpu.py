"""The native reader's way to the device: staging in pieces and conversion there."""
import pytest
import torch

from gguf_rs_cli_b200.weights import SafetensorsFile, TensorSource, WeightFileError, WeightStore, TensorRequest, write_safetensors

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_upload_converts_on_the_device_and_in_pieces(tmp_path):
    g = torch.Generator().manual_seed(3)
    t = {
        "big32": torch.randn(3000, 4100, generator=g),                    # 49 MB: more than one staging buffer
        "big16": torch.randn(5000, 4100, generator=g).to(torch.bfloat16),  # 41 MB, kept as stored
        "half": (torch.randn(257, 33, generator=g) * 100).to(torch.float16),
        "double": torch.randn(1001, generator=g, dtype=torch.float64) * 1e3,
        "i64": torch.randint(-2 ** 31, 2 ** 31 - 1, (777,), generator=g, dtype=torch.int64),
        "i32": torch.randint(-1000, 1000, (5, 7), generator=g, dtype=torch.int32),
        "u8": torch.randint(0, 256, (300,), generator=g, dtype=torch.uint8),
        "i8": torch.randint(-128, 128, (300,), generator=g, dtype=torch.int8),
        "i16": torch.randint(-30000, 30000, (300,), generator=g, dtype=torch.int16),
        "none": torch.empty(0, 8),
    }
    path = str(tmp_path / "w.safetensors")
    write_safetensors(path, t.items())
    f = SafetensorsFile(path)
    for name, v in t.items():
        keeps = (torch.float32, torch.bfloat16) if v.dtype.is_floating_point else (torch.int32,)
        for keep in keeps:
            got = f.to_device(name, keep, DEV)
            assert got.dtype == keep and got.shape == v.shape and got.is_cuda
            want = v.to(torch.float32).to(keep) if v.dtype == torch.float64 else v.to(keep)
            assert torch.equal(got.cpu(), want), f"{name} kept as {keep}"
    with pytest.raises(WeightFileError, match="cannot be kept"):
        f.to_device("i32", torch.float32, DEV)
    with pytest.raises(WeightFileError, match="cannot be kept"):
        f.to_device("half", torch.int32, DEV)
    # several tensors one after the other share the staging buffers
    a = [f.to_device("big32", torch.bfloat16, DEV) for _ in range(3)]
    torch.cuda.synchronize()
    assert all(torch.equal(x, a[0]) for x in a)


def test_store_from_a_folder_keeps_what_the_rules_say(tmp_path):
    w = {"a": torch.randn(64, 8).to(torch.bfloat16), "n": torch.ones(8), "h": torch.randn(3, 8).to(torch.float16),
         "i": torch.arange(9, dtype=torch.int64)}
    (tmp_path / "m").mkdir()
    write_safetensors(str(tmp_path / "m" / "model.safetensors"), w.items())
    for mode in (torch.bfloat16, torch.float32):
        s = WeightStore(TensorSource.from_folder(str(tmp_path / "m")), mode, DEV)
        s.check([TensorRequest("a", (64, 8)), TensorRequest("n", (8,)), TensorRequest("h", (3, 8)), TensorRequest("i", (9,))])
        a, n, h, i = (s.get(TensorRequest(k, tuple(w[k].shape))) for k in "anhi")
        assert a.dtype == mode and n.dtype == torch.float32 and h.dtype == mode and i.dtype == torch.int32
        assert torch.equal(a.cpu(), w["a"].to(mode)) and torch.equal(h.cpu(), w["h"].to(mode))
        assert torch.equal(n.cpu(), w["n"]) and torch.equal(i.cpu(), w["i"].to(torch.int32))

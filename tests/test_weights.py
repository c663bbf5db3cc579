"""Weights by tensor name: file format, kept precision, the one error that lists everything wrong, and
the random-weights mode."""
import json
import os

import pytest
import torch

from helpers import TINY, tiny_config, write_tiny
from iian_b200.config.registry import get_architecture
from iian_b200.engine.model import declare_tensors
from iian_b200.weights.loader import FileWeights, WeightsError, kept_dtype, load_declared
from iian_b200.weights.safetensors_io import SafetensorsError, SafetensorsFile, TensorStore, write_safetensors

ARCH = get_architecture("Qwen3ForCausalLM")


def declared_for(name):
    return declare_tensors(ARCH, ARCH.build_spec(tiny_config(name)))


def test_safetensors_round_trip(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).view(2, 3),
         "d": torch.randn(2, 2).to(torch.float16)}
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, t, {"note": "test"})
    f = SafetensorsFile(path)
    assert f.metadata["note"] == "test" and sorted(f.names()) == ["a", "b", "c", "d"]
    for k, v in t.items():
        got = f.read(k)
        assert got.dtype == v.dtype and got.shape == v.shape and torch.equal(got, v)
    f.close()


def test_the_file_can_be_read_by_the_safetensors_package(tmp_path):
    st = pytest.importorskip("safetensors.torch")
    t = {"w": torch.randn(4, 4).to(torch.bfloat16), "n": torch.ones(4)}
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, t)
    got = st.load_file(path)
    assert all(torch.equal(got[k], t[k]) for k in t)
    st.save_file(t, str(tmp_path / "y.safetensors"))
    f = SafetensorsFile(str(tmp_path / "y.safetensors"))
    assert all(torch.equal(f.read(k), t[k]) for k in t)


def test_broken_files_are_refused(tmp_path):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(b"\x01")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(str(p))
    p.write_bytes((10 ** 9).to_bytes(8, "little") + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(len(hdr).to_bytes(8, "little") + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="data_offsets"):
        SafetensorsFile(str(p))
    with pytest.raises(FileNotFoundError):
        TensorStore(str(tmp_path / "nowhere"))


def test_declarations_follow_the_configuration():
    d = declared_for("B")
    assert d["model.embed_tokens.weight"].shape == (503, 96)
    assert d["lm_head.weight"].shape == (503, 96)
    assert d["model.layers.2.self_attn.q_proj.weight"].shape == (256, 96)
    assert d["model.layers.0.self_attn.k_proj.weight"].shape == (64, 96)
    assert d["model.layers.0.self_attn.o_proj.weight"].shape == (96, 256)
    assert d["model.layers.1.self_attn.q_norm.weight"].shape == (32,)
    assert d["model.layers.1.mlp.down_proj.weight"].shape == (96, 160)
    assert d["model.layers.0.self_attn.q_proj.bias"].optional
    assert "lm_head.weight" not in declared_for("A")            # tied: the head declares nothing


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = write_tiny(tmp_path, "B")
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    tensors = {n: f.read(n) for n in f.names()}
    f.close()
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.9.extra.weight"] = torch.zeros(2)
    tensors["model.layers.0.self_attn.q_norm.weight"] = torch.ones(16)
    tensors["model.embed_tokens.weight"] = torch.zeros(503, 96, dtype=torch.int32)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    src = FileWeights(d)
    with pytest.raises(WeightsError) as ei:
        load_declared(declared_for("B"), src, torch.float32, torch.device("cpu"))
    src.close()
    e = ei.value
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.9.extra.weight"]
    assert e.wrong_shape == [("model.layers.0.self_attn.q_norm.weight", (32,), (16,))]
    assert e.wrong_dtype and e.wrong_dtype[0][0] == "model.embed_tokens.weight"
    msg = str(e)
    for piece in ("missing tensors (2)", "unexpected tensors (1)", "expected [32], got [16]", "model.norm.weight"):
        assert piece in msg


def test_tied_model_with_a_head_in_the_file_is_an_error(tmp_path):
    d = write_tiny(tmp_path, "A")
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    tensors = {n: f.read(n) for n in f.names()}
    f.close()
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    src = FileWeights(d)
    with pytest.raises(WeightsError, match="unexpected tensors .*lm_head.weight"):
        load_declared(declared_for("A"), src, torch.float32, torch.device("cpu"))
    src.close()


def test_kept_precision():
    bf, f32, f16 = torch.bfloat16, torch.float32, torch.float16
    assert kept_dtype(bf, "float", bf) == bf
    assert kept_dtype(f16, "float", bf) == bf
    assert kept_dtype(f32, "float", bf) == f32                  # a tensor stored in 32 bits stays so
    assert kept_dtype(bf, "float", f32) == f32                  # the 32-bit path widens everything
    assert kept_dtype(torch.int64, "int", bf) == torch.int32


def test_loaded_tensors_keep_their_stored_precision(tmp_path):
    d = write_tiny(tmp_path, "B", store_dtype=torch.bfloat16)
    src = FileWeights(d)
    got = load_declared(declared_for("B"), src, torch.bfloat16, torch.device("cpu"))
    src.close()
    assert got["model.layers.0.mlp.gate_proj.weight"].dtype == torch.bfloat16
    assert got["model.layers.0.input_layernorm.weight"].dtype == torch.float32   # the writer stores norm weights in 32 bits
    assert "model.layers.0.self_attn.q_proj.bias" not in got                      # optional and absent
    src = FileWeights(d)
    got32 = load_declared(declared_for("B"), src, torch.float32, torch.device("cpu"))
    src.close()
    assert all(t.dtype == torch.float32 for t in got32.values())
    w16, w32 = got["model.layers.0.mlp.gate_proj.weight"], got32["model.layers.0.mlp.gate_proj.weight"]
    assert torch.equal(w16.float(), w32)                                         # widening is exact


def test_random_weights_mode(tmp_path):
    d1 = write_tiny(tmp_path / "one", "B", seed=3)
    d2 = write_tiny(tmp_path / "two", "B", seed=3)
    d3 = write_tiny(tmp_path / "three", "B", seed=4)
    assert sorted(os.listdir(d1)) == ["config.json", "model.safetensors"]
    a, b, c = (SafetensorsFile(os.path.join(d, "model.safetensors")) for d in (d1, d2, d3))
    assert sorted(a.names()) == sorted(n for n, s in declared_for("B").items() if not s.optional)
    w = "model.layers.2.self_attn.v_proj.weight"
    assert torch.equal(a.read(w), b.read(w)) and not torch.equal(a.read(w), c.read(w))
    x = a.read(w)
    assert abs(x.std().item() - 0.02) < 0.004 and abs(x.mean().item()) < 0.004
    n = a.read("model.layers.0.self_attn.q_norm.weight")
    assert n.dtype == torch.float32 and (n - 1).abs().max() <= 0.1 + 1e-6 and (n - 1).abs().max() > 0.01
    with open(os.path.join(d1, "config.json")) as f:
        assert ARCH.load_config(json.load(f)) == tiny_config("B")
    for f in (a, b, c):
        f.close()


def test_random_values_are_a_function_of_seed_name_and_index():
    """The generator is counter-based: an element depends on (seed, tensor name, index) only -- not on the slab
    it was drawn in, not on other tensors -- and is written out here a second time with Python integers."""
    from iian_b200.weights import random_init as ri
    cpu = torch.device("cpu")
    key = ri.tensor_key(7, "model.layers.0.mlp.up_proj.weight")
    whole = ri.standard_normal(key, 0, 5000, cpu)
    assert torch.equal(whole[1234:1300], ri.standard_normal(key, 1234, 66, cpu))
    assert not torch.equal(whole[:64], ri.standard_normal(ri.tensor_key(7, "model.layers.1.mlp.up_proj.weight"), 0, 64, cpu))
    assert not torch.equal(whole[:64], ri.standard_normal(ri.tensor_key(8, "model.layers.0.mlp.up_proj.weight"), 0, 64, cpu))
    # the same numbers from Python integers (SplitMix64 finaliser, FNV-1a of the name)
    m = (1 << 64) - 1
    def mix(x):
        x = (x + 0x9E3779B97F4A7C15) & m
        x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & m
        x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & m
        return x ^ (x >> 31)
    h = 0xCBF29CE484222325
    for b in b"model.layers.0.mlp.up_proj.weight":
        h = ((h ^ b) * 0x100000001B3) & m
    assert key == mix(7) ^ h
    knots = torch.special.ndtri((torch.arange(65537, dtype=torch.float64) + 0.5) / 65537.0).float()
    for i in (0, 1, 77, 4999):
        bits = mix(((i * 0xD1B54A32D192ED03) & m) ^ key)
        u = bits >> 32
        lo, hi = knots[u >> 16], knots[(u >> 16) + 1]
        want = lo + (hi - lo) * torch.tensor((u & 0xFFFF) / 65536.0, dtype=torch.float32)
        assert whole[i].item() == want.item()
        assert ri.uniform(key, i, 1, cpu).item() == (bits >> 40) / float(1 << 24)
    # and they look normal: mean, variance, fourth moment, tails
    x = ri.standard_normal(key, 0, 1 << 20, cpu).double()
    assert abs(x.mean().item()) < 4e-3 and abs(x.var().item() - 1) < 6e-3 and abs((x ** 4).mean().item() - 3) < 0.05
    assert 0.0024 < (x.abs() > 3).double().mean().item() < 0.0030 and x.abs().max().item() < 4.4
    u = ri.uniform(key, 0, 1 << 20, cpu).double()
    assert abs(u.mean().item() - 0.5) < 2e-3 and abs(u.var().item() - 1 / 12) < 1e-3 and u.min() >= 0 and u.max() < 1


@pytest.mark.gpu
def test_random_values_are_the_same_bits_on_cpu_and_gpu(tmp_path):
    """What lets a plain implementation on the CPU rebuild the model a GPU run drew on the device."""
    from iian_b200.weights import random_init as ri
    from iian_b200.weights.loader import TensorSpec
    for name, spec in (("a.weight", TensorSpec((513, 1031))), ("b.norm", TensorSpec((4099,), init="ones_jitter"))):
        c = ri.draw(name, spec, 11, torch.device("cpu"), 0.02, 0.1)
        g = ri.draw(name, spec, 11, torch.device("cuda:0"), 0.02, 0.1)
        assert torch.equal(c, g.cpu())
    big = TensorSpec(((1 << 24) + 77,))                     # more than one slab
    c = ri.draw("big", big, 3, torch.device("cpu"), 0.02, 0.0)
    g = ri.draw("big", big, 3, torch.device("cuda:0"), 0.02, 0.0)
    assert torch.equal(c, g.cpu())
    from iian_b200.weights.random_init import write_model_folder
    d1 = write_model_folder(str(tmp_path / "c"), ARCH, tiny_config("B"), seed=5)
    d2 = write_model_folder(str(tmp_path / "g"), ARCH, tiny_config("B"), seed=5, device="cuda:0")
    with open(os.path.join(d1, "model.safetensors"), "rb") as f1, open(os.path.join(d2, "model.safetensors"), "rb") as f2:
        assert f1.read() == f2.read()


def test_sharded_folder(tmp_path):
    d = write_tiny(tmp_path, "A")
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    tensors = {n: f.read(n) for n in f.names()}
    f.close()
    os.remove(os.path.join(d, "model.safetensors"))
    names = sorted(tensors)
    half = len(names) // 2
    write_safetensors(os.path.join(d, "model-00001-of-00002.safetensors"), {n: tensors[n] for n in names[:half]})
    write_safetensors(os.path.join(d, "model-00002-of-00002.safetensors"), {n: tensors[n] for n in names[half:]})
    wm = {n: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors") for i, n in enumerate(names)}
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as fh:
        json.dump({"weight_map": wm}, fh)
    src = FileWeights(d)
    got = load_declared(declared_for("A"), src, torch.float32, torch.device("cpu"))
    src.close()
    assert all(torch.equal(got[n], tensors[n].float()) for n in names)
    os.remove(os.path.join(d, "model-00002-of-00002.safetensors"))
    with pytest.raises(FileNotFoundError, match="model-00002"):
        FileWeights(d)

"""Weights: the safetensors container, checks with one clear error, dtype
rules, the random-weights mode."""

import json
import struct

import pytest
import torch

import flashdecode_cuda_b200 as fd
from flashdecode_cuda_b200.engine import Model
from flashdecode_cuda_b200.weights import (SafetensorsError, TensorSpec, WeightError, cast, check, load_checkpoint,
                                           random_tensors, read_file, write_file)
from helpers import TINY, write_folder


def cpu_model(name):
    return Model.from_config(fd.config.config_from_dict(TINY[name]), torch.float32, "cpu")


def test_container_round_trip(tmp_path):
    g = torch.Generator().manual_seed(0)
    tensors = {"a.weight": torch.randn(3, 5, generator=g).to(torch.bfloat16), "b": torch.randn(7, generator=g),
               "ids": torch.arange(6, dtype=torch.int64).view(2, 3), "empty": torch.zeros(0, 4),
               "scalar": torch.tensor(2.5)}
    write_file(tmp_path / "x.safetensors", tensors)
    back = read_file(tmp_path / "x.safetensors")
    assert set(back) == set(tensors)
    for k in tensors:
        assert back[k].dtype == tensors[k].dtype and back[k].shape == tensors[k].shape
        assert torch.equal(back[k], tensors[k])


def test_container_errors(tmp_path):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="shorter"):
        read_file(p)
    p.write_bytes(struct.pack("<Q", 10 ** 9) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        read_file(p)
    p.write_bytes(struct.pack("<Q", 5) + b"hello")
    with pytest.raises(SafetensorsError, match="JSON"):
        read_file(p)
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="offsets"):
        read_file(p)
    with pytest.raises(FileNotFoundError):
        load_checkpoint(tmp_path / "nowhere")


def test_sharded_folder(tmp_path):
    write_file(tmp_path / "s1.safetensors", {"a": torch.ones(2)})
    write_file(tmp_path / "s2.safetensors", {"b": torch.zeros(3)})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}))
    got = load_checkpoint(tmp_path)
    assert set(got) == {"a", "b"} and got["b"].shape == (3,)


def test_specs_name_every_tensor_of_the_checkpoint(tmp_path):
    folder = write_folder(tmp_path, "B")
    names = {s.name for s in cpu_model("B").tensor_specs()}
    assert names == set(load_checkpoint(folder))
    assert "lm_head.weight" in names
    assert "lm_head.weight" not in {s.name for s in cpu_model("A").tensor_specs()}      # tied


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = write_folder(tmp_path, "B")
    tensors = dict(load_checkpoint(folder))
    del tensors["model.layers.1.mlp.up_proj.weight"], tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.o_proj.bias"] = torch.zeros(96)          # the reference refuses it too (loader.py:80-88)
    tensors["model.layers.2.self_attn.q_norm.weight"] = torch.zeros(32)        # Qwen3's per-head norm (loader.py:91-95)
    tensors["model.layers.2.self_attn.k_proj.weight"] = torch.zeros(32, 95)
    tensors["model.embed_tokens.weight"] = torch.zeros(383, 96)
    with pytest.raises(WeightError) as e:
        check(cpu_model("B").tensor_specs(), tensors)
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.o_proj.bias", "model.layers.2.self_attn.q_norm.weight"]
    assert len(err.wrong_shape) == 2 and "expected (32, 96), got (32, 95)" in str(err)
    for word in ("missing", "unexpected", "wrong shapes"):
        assert word in str(err)


def test_biases_optional_or_required_or_refused():
    no_bias = {s.name for s in cpu_model("C").tensor_specs() if not s.optional}
    assert not any(n.endswith("proj.bias") for n in no_bias)
    required = Model.from_config(fd.config.config_from_dict(dict(TINY["A"], attention_bias=True)), torch.float32, "cpu")
    assert any(s.name.endswith("q_proj.bias") and not s.optional for s in required.tensor_specs())
    refused = Model.from_config(fd.config.config_from_dict(dict(TINY["A"], attention_bias=False)), torch.float32, "cpu")
    assert not any(s.name.endswith(".bias") for s in refused.tensor_specs())


def test_dtype_rules():
    m = TensorSpec("w", (2, 2), "matrix")
    v = TensorSpec("n", (2,), "vector")
    t = TensorSpec("ids", (2,), "table")
    bf, f32 = torch.bfloat16, torch.float32
    assert cast(m, torch.ones(2, 2, dtype=bf), bf, "cpu").dtype == bf
    assert cast(m, torch.ones(2, 2, dtype=bf), f32, "cpu").dtype == f32              # 32-bit path: everything 32-bit
    assert cast(v, torch.ones(2, dtype=f32), bf, "cpu").dtype == f32                 # stored in 32-bit stays so
    assert cast(v, torch.ones(2, dtype=bf), bf, "cpu").dtype == bf
    assert cast(t, torch.ones(2, dtype=torch.int64), bf, "cpu").dtype == torch.int32
    assert cast(t, torch.ones(2, dtype=torch.int64), f32, "cpu").dtype == torch.int32


def test_random_weights_depend_on_seed_and_name_only(tmp_path):
    specs = cpu_model("A").tensor_specs()
    a = random_tensors(specs, 5)
    b = random_tensors(list(reversed(specs)), 5)
    c = random_tensors(specs, 6)
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    w = a["model.layers.0.mlp.gate_proj.weight"].float()
    n = a["model.layers.1.input_layernorm.weight"].float()
    assert 0.015 < float(w.std()) < 0.025 and abs(float(w.mean())) < 0.002
    assert 0.9 < float(n.mean()) < 1.1 and 0.05 < float(n.std()) < 0.15
    folder = fd.write_random_model(tmp_path / "m", "tiny-a", 5)
    assert json.loads((folder / "config.json").read_text())["architectures"] == ["Qwen2ForCausalLM"]
    stored = load_checkpoint(folder)
    assert all(t.dtype == torch.bfloat16 for t in stored.values())
    assert torch.equal(stored["model.norm.weight"], a["model.norm.weight"])


def test_no_cpu_path():
    model = cpu_model("A")
    with pytest.raises(RuntimeError, match="CUDA"):
        model.bind(random_tensors(model.tensor_specs(), 0))

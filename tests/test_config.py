"""Configuration: parsing config.json, defaults, refusals, presets, registry."""

import json

import pytest

import flashdecode_cuda_b200 as fd
from flashdecode_cuda_b200.config import ConfigError, Qwen2Config, config_from_dict, load_config, preset_dict, preset_names
from flashdecode_cuda_b200.registry import ARCHITECTURES, architecture, part_class, register_architecture
from helpers import TINY


def test_fields_come_from_config_json():
    cfg = config_from_dict(TINY["C"])
    assert isinstance(cfg, Qwen2Config)
    assert (cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers) == (80, 176, 4)
    assert (cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.num_kv_groups) == (6, 2, 48, 3)
    assert (cfg.vocab_size, cfg.rms_norm_eps, cfg.rope_theta) == (333, 3e-6, 500000.0)
    assert cfg.max_position_embeddings == 512 and cfg.tie_word_embeddings is False
    assert [cfg.layer_window(i) for i in range(4)] == [None, None, 24, 24]


def test_head_dim_defaults_to_hidden_over_heads():
    cfg = config_from_dict(TINY["A"])                # no head_dim key (config.py:122 of the reference)
    assert cfg.head_dim == 64 // 4
    bad = dict(TINY["A"], hidden_size=66)
    with pytest.raises(ConfigError, match="head_dim"):
        config_from_dict(bad)


def test_rope_theta_in_both_layouts():
    flat = config_from_dict(TINY["A"])
    nested = dict(TINY["A"])
    del nested["rope_theta"]
    nested["rope_parameters"] = {"rope_theta": 10000.0, "rope_type": "default"}
    assert config_from_dict(nested).rope_theta == flat.rope_theta
    nested["rope_parameters"] = {"rope_theta": 10000.0, "rope_type": "yarn", "factor": 4.0}
    with pytest.raises(ConfigError, match="yarn"):
        config_from_dict(nested)
    del nested["rope_parameters"]
    with pytest.raises(ConfigError, match="rope_theta"):
        config_from_dict(nested)


@pytest.mark.parametrize("change,match", [
    ({"num_key_value_heads": 3}, "multiple"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"head_dim": 15}, "even"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
    ({"vocab_size": 0}, "positive"),
    ({"use_sliding_window": True}, "sliding_window"),
])
def test_refusals(change, match):
    with pytest.raises(ConfigError, match=match):
        config_from_dict(dict(TINY["A"], **change))


def test_missing_keys_are_listed_together():
    cfg = dict(TINY["B"])
    del cfg["vocab_size"], cfg["rms_norm_eps"]
    with pytest.raises(ConfigError) as e:
        config_from_dict(cfg)
    assert "vocab_size" in str(e.value) and "rms_norm_eps" in str(e.value)


def test_round_trip_and_folder(tmp_path):
    for name in TINY:
        cfg = config_from_dict(TINY[name])
        again = config_from_dict(cfg.to_dict())
        assert again.to_dict() == cfg.to_dict()
    (tmp_path / "config.json").write_text(json.dumps(TINY["B"]))
    assert load_config(tmp_path).hidden_size == 96
    assert load_config(tmp_path / "config.json").vocab_size == 384
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="JSON"):
        load_config(tmp_path)
    with pytest.raises(ConfigError, match="no config.json"):
        load_config(tmp_path / "nowhere")


def test_presets_are_data_and_parse():
    assert {"tiny-a", "tiny-b", "qwen2.5-1.5b", "qwen2.5-7b", "qwen2.5-14b"} <= set(preset_names())
    big = load_config("qwen2.5-1.5b")
    assert (big.num_hidden_layers, big.hidden_size, big.num_kv_groups, big.vocab_size) == (28, 1536, 6, 151936)
    assert load_config("qwen2.5-7b").num_kv_groups == 7 and load_config("qwen2.5-14b").num_kv_groups == 5
    assert preset_dict("tiny-b")["rope_theta"] == 1000000.0


def test_registry_chooses_by_architecture_name():
    assert architecture("Qwen2ForCausalLM").config_cls is Qwen2Config
    with pytest.raises(ConfigError, match="unknown architecture"):
        config_from_dict(dict(TINY["A"], architectures=["NoSuchModel"]))
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict({k: v for k, v in TINY["A"].items() if k != "architectures"})
    with pytest.raises(ValueError, match="already registered"):
        register_architecture("Qwen2ForCausalLM", Qwen2Config, lambda c: None)
    with pytest.raises(KeyError, match="no mixer part"):
        part_class("mixer", "nothing")


def test_blueprint_lists_parts_layer_by_layer():
    cfg = config_from_dict(TINY["C"])
    bp = ARCHITECTURES["Qwen2ForCausalLM"].blueprint(cfg)
    assert len(bp.layers) == 4 and [r.layer for r in bp.schedule] == [0, 1, 2, 3]
    assert [l.mixer.params["window"] for l in bp.layers] == [None, None, 24, 24]
    assert bp.layers[1].mixer.prefix == "model.layers.1.self_attn"
    assert bp.head.params["tied_to"] is None
    tied = ARCHITECTURES["Qwen2ForCausalLM"].blueprint(config_from_dict(TINY["A"]))
    assert tied.head.params["tied_to"] == "model.embed_tokens.weight"


def test_sizes_the_kernels_do_not_take_are_refused_when_the_model_is_built():
    """A head size that is no multiple of 16 passes the configuration (the reference's own tiny model has 8)
    but no attention kernel takes it: the mixer says so when it is built, not at the first step."""
    import torch
    from flashdecode_cuda_b200.engine import Model
    raw = dict(TINY["A"], head_dim=8)
    cfg = config_from_dict(raw)
    with pytest.raises(ValueError, match="head size 8"):
        Model.from_config(cfg, torch.float32, "cpu")
    Model.from_config(config_from_dict(dict(TINY["A"], head_dim=48)), torch.float32, "cpu")


def test_a_layer_is_a_block_name_and_named_parts():
    from flashdecode_cuda_b200.engine import LayerSpec, PartSpec
    n = lambda p: PartSpec("norm", "rmsnorm", dict(size=8, eps=1e-5), p)
    by_position = LayerSpec("prenorm", n("a"), PartSpec("mixer", "x"), n("b"), PartSpec("feed_forward", "y"))
    by_name = LayerSpec("prenorm", norm1=n("a"), mixer=PartSpec("mixer", "x"), norm2=n("b"), feed_forward=PartSpec("feed_forward", "y"))
    assert list(by_position.parts) == list(by_name.parts) == ["norm1", "mixer", "norm2", "feed_forward"]
    assert by_position.mixer.name == "x" and by_name.norm2.prefix == "b"
    free = LayerSpec("anything", {"only_norm": n("c")}, extra=n("d"))
    assert list(free.parts) == ["only_norm", "extra"]
    with pytest.raises(TypeError):
        LayerSpec("prenorm", norm1="not a spec")
    with pytest.raises(AttributeError):
        by_name.norm3

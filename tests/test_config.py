"""Configuration and registry."""
import json

import pytest

from rvllm_b200.config import Lfm2Config, config_from_dict, load_config, registered_architectures
from rvllm_b200.errors import ConfigError
from tiny import TINY_A, TINY_B, tiny

PUBLISHED = {   # block_ff_dim -> adjusted, from the published sizes
    12288: 8192, 6656: 4608, 10240: 6912,
}


def test_tiny_configs_parse_and_differ():
    a, b = config_from_dict(tiny("A")), config_from_dict(tiny("B"))
    assert a.layer_kinds == ["conv", "full_attention", "conv", "full_attention"]
    assert b.layer_kinds == ["conv", "conv", "full_attention", "conv", "conv", "full_attention"]
    assert (a.ffn_dim, b.ffn_dim) == (192, 256)
    assert (a.group_size, b.group_size) == (2, 3)
    for field in ("num_hidden_layers", "hidden_size", "num_attention_heads",
                  "num_key_value_heads", "head_dim", "vocab_size", "max_position_embeddings",
                  "norm_eps", "rope_theta", "conv_L_cache", "conv_bias", "tie_embedding"):
        assert getattr(a, field) != getattr(b, field), field


@pytest.mark.parametrize("ff,want", sorted(PUBLISHED.items()))
def test_feed_forward_adjustment(ff, want):
    d = tiny("A")
    d.update(block_ff_dim=ff, block_auto_adjust_ff_dim=True, block_multiple_of=256)
    assert config_from_dict(d).ffn_dim == want


def test_multiplier_applies_before_rounding():
    d = tiny("A")
    d.update(block_ff_dim=300, block_auto_adjust_ff_dim=True, block_multiple_of=64,
             block_ffn_dim_multiplier=1.5)
    assert config_from_dict(d).ffn_dim == 320      # int(2*300/3)=200 -> 300 -> 320


def test_layer_types_instead_of_indices():
    d = tiny("A")
    del d["full_attn_idxs"]
    d["layer_types"] = ["conv", "full_attention", "conv", "full_attention"]
    assert config_from_dict(d).full_attn_idxs == (1, 3)


def test_head_dim_defaults_to_hidden_over_heads():
    d = tiny("A")
    del d["head_dim"]
    assert config_from_dict(d).head_dim == 16


def test_round_trip():
    for name in ("A", "B"):
        cfg = config_from_dict(tiny(name))
        assert config_from_dict(cfg.to_dict()) == cfg


@pytest.mark.parametrize("key", ["num_hidden_layers", "hidden_size", "num_attention_heads",
                                 "num_key_value_heads", "vocab_size", "norm_eps", "rope_theta",
                                 "max_position_embeddings", "block_ff_dim", "conv_L_cache",
                                 "block_auto_adjust_ff_dim"])
def test_missing_key_is_named(key):
    d = tiny("B")
    del d[key]
    with pytest.raises(ConfigError, match=key):
        config_from_dict(d)


@pytest.mark.parametrize("key,value", [("hidden_size", "64"), ("norm_eps", "small"),
                                        ("conv_bias", 1), ("full_attn_idxs", [1, "3"]),
                                        ("num_hidden_layers", 2.5)])
def test_wrong_type_is_named(key, value):
    d = tiny("A")
    d[key] = value
    with pytest.raises(ConfigError, match=key):
        config_from_dict(d)


@pytest.mark.parametrize("change,message", [
    ({"num_attention_heads": 4, "num_key_value_heads": 3}, "invalid attention head counts"),
    ({"head_dim": 15}, "must be even"),
    ({"full_attn_idxs": [1, 4]}, "out of range"),
    ({"full_attn_idxs": [3, 1]}, "sorted and unique"),
    ({"full_attn_idxs": []}, "no attention layers"),
    ({"conv_L_cache": 0}, "conv_L_cache"),
    ({"block_auto_adjust_ff_dim": True}, "block_multiple_of"),
    ({"layer_types": ["conv"], "full_attn_idxs": None}, "entries for 4 layers"),
])
def test_contradictions_are_refused(change, message):
    d = tiny("A")
    d.update(change)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(d)


def test_unknown_architecture_lists_the_known_ones():
    d = tiny("A")
    d["architectures"] = ["LlamaForCausalLM"]
    with pytest.raises(ConfigError, match="Lfm2ForCausalLM"):
        config_from_dict(d)
    assert "Lfm2ForCausalLM" in registered_architectures()


def test_missing_architectures_key():
    d = tiny("A")
    del d["architectures"]
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict(d)


def test_load_config_from_folder(tmp_path):
    with pytest.raises(ConfigError, match="config.json"):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    assert isinstance(load_config(str(tmp_path)), Lfm2Config)
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        load_config(str(tmp_path))


def test_spec_follows_the_config():
    from rvllm_b200.config import architecture
    from rvllm_b200.parts.model import param_decls
    cfg = config_from_dict(tiny("B"))
    spec = architecture(cfg.architecture).build_spec(cfg)
    kinds = [b.mixer.kind for b in spec.layers]
    assert kinds == ["short_conv", "short_conv", "attention", "short_conv", "short_conv", "attention"]
    decls = param_decls(spec)
    assert decls["model.layers.0.conv.in_proj.weight"].shape == (288, 96)
    assert decls["model.layers.0.conv.conv.weight"].shape == (96, 4)
    assert decls["model.layers.0.conv.in_proj.bias"].shape == (288,)
    assert decls["model.layers.2.self_attn.k_proj.weight"].shape == (32, 96)
    assert decls["model.layers.2.self_attn.q_layernorm.weight"].shape == (32,)
    assert decls["model.layers.5.feed_forward.w1.weight"].shape == (256, 96)
    assert decls["lm_head.weight"].shape == (1000, 96)
    assert "lm_head.weight" not in param_decls(
        architecture(cfg.architecture).build_spec(config_from_dict(tiny("A"))))

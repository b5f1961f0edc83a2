"""The weights loader: by-name reading, dtype policy, one error for everything wrong,
and the random-weights mode."""
import json
import os

import pytest
import torch

from rvllm_b200.config import architecture, config_from_dict
from rvllm_b200.errors import WeightsError
from rvllm_b200.parts.model import param_decls
from rvllm_b200.weights import (SafetensorsFile, load_tensors, random_tensors,
                                write_random_model, write_safetensors)
from tiny import tiny, write_tiny


def spec_of(name):
    cfg = config_from_dict(tiny(name))
    return cfg, architecture(cfg.architecture).build_spec(cfg)


def test_random_model_folder_round_trip(tmp_path):
    folder = write_tiny(str(tmp_path), "B")
    assert sorted(os.listdir(folder)) == ["config.json", "model.safetensors"]
    cfg, spec = spec_of("B")
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    assert set(f.names()) == set(param_decls(spec))
    assert all(f.dtype(n) == torch.bfloat16 for n in f.names())
    w = load_tensors(folder, spec, torch.bfloat16, "cpu")
    again = random_tensors(cfg, 1)
    for n, t in w.items():
        assert t.dtype == torch.bfloat16 and torch.equal(t, again[n]), n


def test_random_weights_follow_the_stated_distributions(tmp_path):
    cfg, _ = spec_of("B")
    w = {n: t.float() for n, t in random_tensors(cfg, 3).items()}
    lin = w["model.layers.0.feed_forward.w1.weight"]
    assert abs(float(lin.std()) - 0.02) < 0.002 and abs(float(lin.mean())) < 0.002
    conv = w["model.layers.0.conv.conv.weight"]
    assert abs(float(conv.std()) - 0.2) < 0.05
    norm = w["model.layers.3.ffn_norm.weight"]
    assert abs(float(norm.mean()) - 1.0) < 0.03 and 0.02 < float(norm.std()) < 0.08
    # another seed, other values; same seed, same values; a tensor does not depend on the rest
    assert not torch.equal(random_tensors(cfg, 4)["lm_head.weight"], random_tensors(cfg, 3)["lm_head.weight"])
    a_cfg, _ = spec_of("A")
    assert a_cfg.hidden_size != cfg.hidden_size


def test_float32_mode_widens_exactly(tmp_path):
    folder = write_tiny(str(tmp_path), "A")
    _, spec = spec_of("A")
    w32 = load_tensors(folder, spec, torch.float32, "cpu")
    w16 = load_tensors(folder, spec, torch.bfloat16, "cpu")
    for n in w32:
        assert w32[n].dtype == torch.float32 and torch.equal(w32[n], w16[n].float())


def test_a_tensor_stored_in_32_bits_stays_so(tmp_path):
    folder = write_tiny(str(tmp_path), "A")
    _, spec = spec_of("A")
    path = os.path.join(folder, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    name32 = "model.layers.1.self_attn.q_layernorm.weight"
    name16 = "model.layers.0.operator_norm.weight"
    tensors[name32] = tensors[name32].float() + 1e-4          # not representable in bfloat16
    tensors["model.layers.1.ffn_norm.weight"] = tensors["model.layers.1.ffn_norm.weight"].half()
    del f
    write_safetensors(path, tensors)
    w = load_tensors(folder, spec, torch.bfloat16, "cpu")
    assert w[name32].dtype == torch.float32 and torch.equal(w[name32], tensors[name32])
    assert w[name16].dtype == torch.bfloat16
    assert w["model.layers.1.ffn_norm.weight"].dtype == torch.bfloat16   # float16 narrows


def test_conv_filter_stored_with_a_unit_axis(tmp_path):
    folder = write_tiny(str(tmp_path), "A")
    cfg, spec = spec_of("A")
    path = os.path.join(folder, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    name = "model.layers.0.conv.conv.weight"
    flat = tensors[name].clone()
    tensors[name] = flat.reshape(cfg.hidden_size, 1, cfg.conv_L_cache)
    del f
    write_safetensors(path, tensors)
    w = load_tensors(folder, spec, torch.bfloat16, "cpu")
    assert w[name].shape == (cfg.hidden_size, cfg.conv_L_cache) and torch.equal(w[name], flat)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = write_tiny(str(tmp_path), "B")
    _, spec = spec_of("B")
    path = os.path.join(folder, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    del f
    del tensors["model.layers.2.self_attn.k_proj.weight"]
    del tensors["lm_head.weight"]
    tensors["model.layers.9.extra.weight"] = torch.zeros(3)
    tensors["model.embedding_norm.weight"] = torch.zeros(95, dtype=torch.bfloat16)
    tensors["model.layers.0.conv.in_proj.weight"] = torch.zeros(96, 288, dtype=torch.bfloat16)
    write_safetensors(path, tensors)
    with pytest.raises(WeightsError) as e:
        load_tensors(folder, spec, torch.bfloat16, "cpu")
    msg = str(e.value)
    assert "missing tensors (2): lm_head.weight, model.layers.2.self_attn.k_proj.weight" in msg
    assert "unexpected tensors (1): model.layers.9.extra.weight" in msg
    assert "wrong shapes (2)" in msg
    assert "model.embedding_norm.weight has [95], expected [96]" in msg
    assert "model.layers.0.conv.in_proj.weight has [96, 288], expected [288, 96]" in msg


def test_missing_file_and_broken_file(tmp_path):
    _, spec = spec_of("A")
    with pytest.raises(WeightsError, match="model.safetensors"):
        load_tensors(str(tmp_path), spec, torch.bfloat16, "cpu")
    (tmp_path / "model.safetensors").write_bytes(b"\xff" * 4)
    with pytest.raises(ValueError, match="too short"):
        load_tensors(str(tmp_path), spec, torch.bfloat16, "cpu")
    (tmp_path / "model.safetensors").write_bytes((10 ** 9).to_bytes(8, "little") + b"{}")
    with pytest.raises(ValueError, match="header length"):
        load_tensors(str(tmp_path), spec, torch.bfloat16, "cpu")


def test_sharded_folder_with_an_index(tmp_path):
    folder = write_tiny(str(tmp_path), "A")
    _, spec = spec_of("A")
    path = os.path.join(folder, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    del f
    os.remove(path)
    names = sorted(tensors)
    parts = {"model-00001-of-00002.safetensors": names[:7], "model-00002-of-00002.safetensors": names[7:]}
    for fn, ns in parts.items():
        write_safetensors(os.path.join(folder, fn), {n: tensors[n] for n in ns})
    with open(os.path.join(folder, "model.safetensors.index.json"), "w") as fh:
        json.dump({"weight_map": {n: fn for fn, ns in parts.items() for n in ns}}, fh)
    w = load_tensors(folder, spec, torch.bfloat16, "cpu")
    assert all(torch.equal(w[n], tensors[n]) for n in names)

"""Configuration, registry and weight loading: what is accepted, what is refused, and
that one error names everything that is wrong."""
from __future__ import annotations

import json
import os

import pytest
import torch

from conftest import TINY
from toyinfer_b200 import models  # noqa: F401
from toyinfer_b200.config import (ConfigError, Qwen3Config, load_config, register_architecture,
                                  registered_architectures, resolve_architecture, unregister_architecture)
from toyinfer_b200.parts.model import DecoderModel
from toyinfer_b200.weights import (SafetensorsFile, WeightError, load_parameters, write_model_folder,
                                   write_safetensors)


def test_config_reads_every_key():
    c = Qwen3Config.from_dict(dict(TINY["B"]))
    assert (c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (96, 6, 2, 32)
    assert c.q_dim == 192 and c.kv_dim == 64
    assert c.stop_token_ids == (11, 12)
    assert c.tie_word_embeddings is False and c.rms_norm_eps == 1e-5 and c.rope_theta == 1e6
    assert [c.layer_window(i) for i in range(3)] == [0, 0, 0]


def test_config_defaults_and_window():
    raw = dict(TINY["A"])
    del raw["head_dim"]
    c = Qwen3Config.from_dict(raw)
    assert c.head_dim == 16 and c.stop_token_ids == (7,)
    c = Qwen3Config.from_dict(dict(TINY["C"]))
    assert [c.layer_window(i) for i in range(4)] == [0, 40, 40, 40]
    raw = dict(TINY["C"], layer_types=["sliding_attention", "full_attention", "full_attention", "sliding_attention"])
    assert [Qwen3Config.from_dict(raw).layer_window(i) for i in range(4)] == [40, 0, 0, 40]


def test_config_errors_are_collected():
    raw = dict(TINY["A"])
    del raw["vocab_size"], raw["rope_theta"]
    raw["hidden_size"] = "64"
    with pytest.raises(ConfigError) as e:
        Qwen3Config.from_dict(raw)
    msg = str(e.value)
    assert "vocab_size: missing" in msg and "rope_theta: missing" in msg and "hidden_size: expected an integer" in msg


@pytest.mark.parametrize("change,needle", [
    ({"num_key_value_heads": 3}, "multiple"), ({"head_dim": 15}, "even"), ({"hidden_act": "gelu"}, "silu"),
    ({"attention_bias": True}, "bias"), ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"),
    ({"use_sliding_window": True}, "sliding_window"), ({"num_hidden_layers": 0}, "positive"),
    ({"layer_types": ["full_attention"]}, "layer_types"),
])
def test_config_refuses(change, needle):
    with pytest.raises(ConfigError) as e:
        Qwen3Config.from_dict(dict(TINY["A"], **change))
    assert needle in str(e.value)


def test_registry(tmp_path):
    assert "Qwen3ForCausalLM" in registered_architectures()
    with pytest.raises(ConfigError) as e:
        resolve_architecture("NoSuchModel")
    assert "Qwen3ForCausalLM" in str(e.value)
    (tmp_path / "config.json").write_text(json.dumps(dict(TINY["A"], architectures=["Other"])))
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))
    register_architecture("Other", Qwen3Config, resolve_architecture("Qwen3ForCausalLM").describe)
    try:
        arch, cfg = load_config(str(tmp_path))
        assert arch.name == "Other" and cfg.hidden_size == 64
        with pytest.raises(ValueError):
            register_architecture("Other", Qwen3Config, None)
    finally:
        unregister_architecture("Other")
    with pytest.raises(ConfigError):
        load_config(str(tmp_path / "missing"))


def _model(name, dtype=torch.float32):
    arch = resolve_architecture("Qwen3ForCausalLM")
    return DecoderModel(arch.describe(Qwen3Config.from_dict(dict(TINY[name]))), dtype, "cpu")


def test_random_folder_roundtrip(model_folders):
    for name in TINY:
        m = _model(name)
        specs = m.param_specs()
        t = load_parameters(specs, model_folders[name], torch.float32, "cpu", m.ignorable_names())
        assert set(t) == set(specs)
        for n, s in specs.items():
            assert tuple(t[n].shape) == s.shape and t[n].dtype == torch.float32
        norm = t["model.norm.weight"]
        assert abs(norm.mean().item() - 1) < 0.05 and 0.005 < t["model.layers.0.mlp.up_proj.weight"].std().item() < 0.04
        b = load_parameters(specs, model_folders[name], torch.bfloat16, "cpu", m.ignorable_names())
        assert all(x.dtype == torch.bfloat16 for x in b.values())
        assert torch.equal(b["model.norm.weight"].float(), norm)           # the file holds bfloat16 values
    assert ("lm_head.weight" in _model("B").param_specs()) and ("lm_head.weight" not in _model("A").param_specs())


def test_same_seed_same_weights(tmp_path):
    a = write_model_folder(dict(TINY["A"]), 5, str(tmp_path / "a"))
    b = write_model_folder(dict(TINY["A"]), 5, str(tmp_path / "b"))
    c = write_model_folder(dict(TINY["A"]), 6, str(tmp_path / "c"))
    fa, fb, fc = (SafetensorsFile(os.path.join(d, "model.safetensors")) for d in (a, b, c))
    n = "model.layers.1.self_attn.k_proj.weight"
    assert torch.equal(fa.tensor(n), fb.tensor(n)) and not torch.equal(fa.tensor(n), fc.tensor(n))


def test_one_error_lists_missing_unexpected_and_wrong(tmp_path, model_folders):
    m = _model("A")
    src = SafetensorsFile(os.path.join(model_folders["A"], "model.safetensors"))
    tensors = {n: src.tensor(n).clone() for n in src.entries}
    del tensors["model.layers.0.mlp.up_proj.weight"], tensors["model.norm.weight"]
    tensors["model.layers.1.self_attn.q_proj.weight"] = torch.zeros(64, 60, dtype=torch.bfloat16)
    tensors["model.layers.7.extra.weight"] = torch.zeros(3, dtype=torch.bfloat16)
    tensors["model.layers.1.input_layernorm.weight"] = torch.zeros(64, dtype=torch.int32)
    d = tmp_path / "bad"
    d.mkdir()
    write_safetensors(str(d / "model.safetensors"), tensors.items())
    with pytest.raises(WeightError) as e:
        load_parameters(m.param_specs(), str(d), torch.float32, "cpu", m.ignorable_names())
    msg = str(e.value)
    assert "missing tensors (2)" in msg and "model.layers.0.mlp.up_proj.weight" in msg and "model.norm.weight" in msg
    assert "unexpected tensors (1)" in msg and "model.layers.7.extra.weight" in msg
    assert "[64, 60]" in msg and "[64, 64]" in msg
    assert "model.layers.1.input_layernorm.weight" in msg


def test_32_bit_tensors_are_not_narrowed(tmp_path, model_folders):
    m = _model("A")
    src = SafetensorsFile(os.path.join(model_folders["A"], "model.safetensors"))
    tensors = {n: src.tensor(n).clone() for n in src.entries}
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float() + 1e-4       # not a bfloat16 value
    d = tmp_path / "f32norm"
    d.mkdir()
    write_safetensors(str(d / "model.safetensors"), tensors.items())
    t = load_parameters(m.param_specs(), str(d), torch.bfloat16, "cpu", m.ignorable_names())
    assert t["model.norm.weight"].dtype == torch.float32
    assert torch.equal(t["model.norm.weight"], tensors["model.norm.weight"])
    assert t["model.embed_tokens.weight"].dtype == torch.bfloat16
    tensors["model.layers.0.mlp.up_proj.weight"] = tensors["model.layers.0.mlp.up_proj.weight"].float()
    write_safetensors(str(d / "model.safetensors"), tensors.items())
    with pytest.raises(WeightError) as e:
        load_parameters(m.param_specs(), str(d), torch.bfloat16, "cpu", m.ignorable_names())
    assert "float32" in str(e.value)
    t = load_parameters(m.param_specs(), str(d), torch.float32, "cpu", m.ignorable_names())
    assert t["model.layers.0.mlp.up_proj.weight"].dtype == torch.float32


def test_tied_checkpoint_may_carry_a_head(tmp_path, model_folders):
    m = _model("A")
    src = SafetensorsFile(os.path.join(model_folders["A"], "model.safetensors"))
    tensors = {n: src.tensor(n).clone() for n in src.entries}
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    d = tmp_path / "tied"
    d.mkdir()
    write_safetensors(str(d / "model.safetensors"), tensors.items())
    load_parameters(m.param_specs(), str(d), torch.float32, "cpu", m.ignorable_names())


def test_truncated_and_sharded_files(tmp_path, model_folders):
    path = os.path.join(model_folders["A"], "model.safetensors")
    raw = open(path, "rb").read()
    d = tmp_path / "cut"
    d.mkdir()
    (d / "model.safetensors").write_bytes(raw[: len(raw) - 100])
    m = _model("A")
    with pytest.raises(WeightError) as e:
        load_parameters(m.param_specs(), str(d), torch.float32, "cpu")
    assert "truncated" in str(e.value)
    # two shards with an index
    src = SafetensorsFile(path)
    names = sorted(src.entries)
    s = tmp_path / "shards"
    s.mkdir()
    half = len(names) // 2
    write_safetensors(str(s / "model-00001-of-00002.safetensors"), [(n, src.tensor(n)) for n in names[:half]])
    write_safetensors(str(s / "model-00002-of-00002.safetensors"), [(n, src.tensor(n)) for n in names[half:]])
    wm = {n: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
          for i, n in enumerate(names)}
    (s / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    t = load_parameters(m.param_specs(), str(s), torch.float32, "cpu")
    assert torch.equal(t[names[0]], src.tensor(names[0]).float())

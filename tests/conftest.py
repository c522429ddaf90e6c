"""Shared fixtures: tiny configurations, model folders with random weights, markers."""
from __future__ import annotations

import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Tiny configurations that differ in every size and option.
TINY = {
    # heads 4 over 2 kv heads of 16, q_dim == hidden, tied head, theta 1e4, eps 1e-6
    "A": {
        "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 64,
        "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 128,
        "vocab_size": 256, "rope_theta": 1e4, "rms_norm_eps": 1e-6, "max_position_embeddings": 128,
        "tie_word_embeddings": True, "eos_token_id": 7, "bos_token_id": 1,
    },
    # heads 6 over 2 kv heads of 32, q_dim 192 != hidden 96, untied head, theta 1e6, eps 1e-5
    "B": {
        "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 3, "hidden_size": 96,
        "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 32, "intermediate_size": 200,
        "vocab_size": 384, "rope_theta": 1e6, "rms_norm_eps": 1e-5, "max_position_embeddings": 256,
        "tie_word_embeddings": False, "eos_token_id": [11, 12],
    },
    # one kv head of 48 for 5 heads, odd sizes, a window of 40 on the layers above the first
    "C": {
        "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 4, "hidden_size": 80,
        "num_attention_heads": 5, "num_key_value_heads": 1, "head_dim": 48, "intermediate_size": 144,
        "vocab_size": 300, "rope_theta": 5e5, "rms_norm_eps": 3e-6, "max_position_embeddings": 320,
        "tie_word_embeddings": False, "use_sliding_window": True, "sliding_window": 40,
        "max_window_layers": 1,
    },
    # heads of 128 (the size the bfloat16 tensor-core attention kernels take), 4 over 2 kv heads
    "D": {
        "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 256,
        "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 320,
        "vocab_size": 520, "rope_theta": 1e6, "rms_norm_eps": 1e-6, "max_position_embeddings": 1280,
        "tie_word_embeddings": False, "eos_token_id": 3,
    },
    # heads of 64, 6 over 3 kv heads, a window of 64 (a ring with no slack) on the second layer
    "E": {
        "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 192,
        "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 64, "intermediate_size": 136,
        "vocab_size": 410, "rope_theta": 1e5, "rms_norm_eps": 1e-5, "max_position_embeddings": 512,
        "tie_word_embeddings": True, "layer_types": ["full_attention", "sliding_attention"], "sliding_window": 64,
    },
}
SEEDS = {"A": 11, "B": 22, "C": 33, "D": 44, "E": 55}


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """name -> folder with config.json and model.safetensors (bfloat16 values)."""
    from toyinfer_b200.weights import write_model_folder

    out = {}
    for name, cfg in TINY.items():
        d = tmp_path_factory.mktemp(f"tiny_{name}")
        write_model_folder(dict(cfg), SEEDS[name], str(d))
        out[name] = str(d)
    return out


def prompts_for(name: str, lengths, seed: int = 0):
    g = torch.Generator().manual_seed(1000 + seed)
    v = TINY[name]["vocab_size"]
    return [torch.randint(0, v, (n,), generator=g).tolist() for n in lengths]

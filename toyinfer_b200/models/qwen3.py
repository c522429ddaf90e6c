"""Qwen3 dense: the description of the model in terms of parts.

Every layer is a pre-norm block of RMS norm, grouped-query attention with per-head
q/k norm and half-rotation rotary encoding, and a SwiGLU feed-forward; tensor names
are the checkpoint's (src/qwen.cpp:18-29, :415).  Layers the configuration gives a
window get it as a parameter of their mixer.  Nothing here computes: the parts do.
"""
from __future__ import annotations

from ..config.qwen3 import Qwen3Config
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from ..parts.model import LayerSpec, ModelSpec


def describe_qwen3(cfg: Qwen3Config) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps})
    ffn = PartSpec("swiglu", {"intermediate_size": cfg.intermediate_size})
    layers = []
    for i in range(cfg.num_hidden_layers):
        mixer = PartSpec(
            "gqa_attention",
            {
                "n_heads": cfg.num_attention_heads,
                "n_kv_heads": cfg.num_key_value_heads,
                "head_dim": cfg.head_dim,
                "qk_norm_eps": cfg.rms_norm_eps,
                "position": "rope",
                "window": cfg.layer_window(i),
            },
        )
        block = PartSpec("prenorm", {"norm": norm, "mixer": mixer, "feed_forward": ffn})
        layers.append(LayerSpec(prefix=f"model.layers.{i}.", block=block))
    return ModelSpec(
        vocab_size=cfg.vocab_size,
        hidden_size=cfg.hidden_size,
        max_positions=cfg.max_position_embeddings,
        layers=layers,
        final_norm=norm,
        positions={
            "rope": PartSpec(
                "rotary_half",
                {"dim": cfg.head_dim, "theta": cfg.rope_theta, "max_positions": cfg.max_position_embeddings},
            )
        },
        tie_head=cfg.tie_word_embeddings,
        stop_token_ids=cfg.stop_token_ids,
    )


register_architecture("Qwen3ForCausalLM", Qwen3Config, describe_qwen3)

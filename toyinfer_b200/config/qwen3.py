"""Configuration of the Qwen3 dense decoder, from its own config.json keys.

The reference reads vocab_size, hidden_size, intermediate_size, num_hidden_layers,
num_attention_heads, num_key_value_heads, head_dim, bos_token_id, eos_token_id,
max_position_embeddings, rms_norm_eps and rope_theta (src/config.cpp:26-37) and
requires an even head_dim (src/config.cpp:39-41).  It ignores
tie_word_embeddings (the head is always the embedding table, src/qwen.cpp:482-483),
hidden_act (SiLU is hard-coded, src/decode.cu:756-762), attention_bias,
rope_scaling and the sliding-window keys.  Here those keys are read too: the ones
this engine implements select behaviour (tied head, window per layer) and the
ones it does not implement are refused instead of ignored.
"""
from __future__ import annotations

from typing import List, Optional

from .base import Key, ModelConfig

FULL = "full_attention"
SLIDING = "sliding_attention"


class Qwen3Config(ModelConfig):
    KEYS = {
        "architectures": Key("str_list", required=False, default=("Qwen3ForCausalLM",)),
        "vocab_size": Key("int"),
        "hidden_size": Key("int"),
        "intermediate_size": Key("int"),
        "num_hidden_layers": Key("int"),
        "num_attention_heads": Key("int"),
        "num_key_value_heads": Key("int"),
        "head_dim": Key(
            "int",
            required=False,
            default=lambda v: v["hidden_size"] // v["num_attention_heads"],
        ),
        "max_position_embeddings": Key("int"),
        "rms_norm_eps": Key("float"),
        "rope_theta": Key("float"),
        "tie_word_embeddings": Key("bool", required=False, default=False),
        "bos_token_id": Key("int", required=False, default=None, nullable=True),
        "eos_token_id": Key("int_or_list", required=False, default=(), nullable=True),
        "hidden_act": Key("str", required=False, default="silu"),
        "attention_bias": Key("bool", required=False, default=False),
        "rope_scaling": Key("any", required=False, default=None, nullable=True),
        "use_sliding_window": Key("bool", required=False, default=False),
        "sliding_window": Key("int", required=False, default=None, nullable=True),
        "max_window_layers": Key(
            "int", required=False, default=lambda v: v["num_hidden_layers"]
        ),
        "layer_types": Key("str_list", required=False, default=None, nullable=True),
    }

    def validate(self) -> List[str]:
        p: List[str] = []
        for name in (
            "vocab_size",
            "hidden_size",
            "intermediate_size",
            "num_hidden_layers",
            "num_attention_heads",
            "num_key_value_heads",
            "head_dim",
            "max_position_embeddings",
        ):
            if getattr(self, name) <= 0:
                p.append(f"{name}: must be positive, got {getattr(self, name)}")
        if p:
            return p
        if self.num_attention_heads % self.num_key_value_heads != 0:
            p.append(
                "num_attention_heads must be a multiple of num_key_value_heads "
                f"({self.num_attention_heads} vs {self.num_key_value_heads})"
            )
        if self.head_dim % 2 != 0:
            p.append(f"head_dim: must be even for half-rotation RoPE, got {self.head_dim}")
        if not (self.rms_norm_eps > 0.0):
            p.append(f"rms_norm_eps: must be positive, got {self.rms_norm_eps}")
        if not (self.rope_theta > 0.0):
            p.append(f"rope_theta: must be positive, got {self.rope_theta}")
        if self.hidden_act != "silu":
            p.append(f"hidden_act: only 'silu' is implemented, got {self.hidden_act!r}")
        if self.attention_bias:
            p.append("attention_bias: projections with bias are not implemented")
        if self.rope_scaling is not None:
            p.append("rope_scaling: scaled rotary embeddings are not implemented")
        if self.eos_token_id is None:
            self.eos_token_id = ()
            self._values["eos_token_id"] = ()
        if self.use_sliding_window and (self.sliding_window is None or self.sliding_window <= 0):
            p.append("use_sliding_window is true but sliding_window is not a positive integer")
        if self.layer_types is not None:
            if len(self.layer_types) != self.num_hidden_layers:
                p.append(
                    f"layer_types: {len(self.layer_types)} entries for "
                    f"{self.num_hidden_layers} layers"
                )
            for t in self.layer_types:
                if t not in (FULL, SLIDING):
                    p.append(f"layer_types: unknown layer type {t!r}")
            if SLIDING in self.layer_types and not (self.sliding_window and self.sliding_window > 0):
                p.append("layer_types names sliding_attention but sliding_window is not set")
        return p

    # -- derived ------------------------------------------------------------
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def layer_window(self, layer: int) -> int:
        """Window of a layer in tokens; 0 means every earlier key is visible.

        ``layer_types`` decides when present.  Otherwise ``use_sliding_window``
        switches the window on for layers with index >= ``max_window_layers``
        (the lower layers keep full attention).  A query at position p sees the
        keys at positions p-window+1 .. p.
        """
        if self.layer_types is not None:
            return int(self.sliding_window) if self.layer_types[layer] == SLIDING else 0
        if self.use_sliding_window and layer >= self.max_window_layers:
            return int(self.sliding_window)
        return 0

    @property
    def stop_token_ids(self) -> tuple:
        return tuple(self.eos_token_id)

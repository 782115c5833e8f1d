"""Typed Qwen3 configuration read from the architecture's own ``config.json`` keys.

Upstream reads thirteen keys and pins every one of them to the 4B checkpoint
(src/forge_engine/qwen3.py:36-88).  Here the same keys are read, none is pinned,
and a few that upstream insists on may be left out where a default is unambiguous.
"""

from __future__ import annotations

import json
import math
from dataclasses import dataclass
from pathlib import Path

from ..errors import ConfigError
from .specs import (
    AttentionSpec,
    GatedMLPSpec,
    LayerSpec,
    ModelSpec,
    NormSpec,
    RotarySpec,
    RunSpec,
)


def _require(raw: dict, key: str):
    if key not in raw:
        raise ConfigError(f"config.json has no key {key!r}")
    return raw[key]


def _positive_int(raw: dict, key: str) -> int:
    value = _require(raw, key)
    if isinstance(value, bool) or not isinstance(value, int) or value < 1:
        raise ConfigError(f"config.json {key}={value!r} must be a positive integer")
    return value


@dataclass(frozen=True)
class Qwen3Config:
    """Sizes and constants of a Qwen3 dense decoder (src/forge_engine/qwen3.py:18-34)."""

    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    eos_token_ids: tuple
    tie_word_embeddings: bool
    attention_bias: bool
    sliding_window: int | None = None
    max_window_layers: int | None = None

    architecture = "Qwen3ForCausalLM"

    # -- reading ----------------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: dict) -> "Qwen3Config":
        model_type = raw.get("model_type", "qwen3")
        if model_type != "qwen3":
            raise ConfigError(f"model_type={model_type!r}; this configuration reads 'qwen3'")
        act = raw.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act={act!r}; Qwen3 uses 'silu'")
        scaling = raw.get("rope_scaling")
        if scaling not in (None, {}) and scaling.get("rope_type", scaling.get("type")) != "default":
            raise ConfigError(f"rope_scaling={scaling!r} is not supported (plain rotary only)")
        hidden = _positive_int(raw, "hidden_size")
        heads = _positive_int(raw, "num_attention_heads")
        kv_heads = _positive_int(raw, "num_key_value_heads")
        head_dim = raw.get("head_dim")
        if head_dim is None:
            if hidden % heads:
                raise ConfigError("head_dim is absent and hidden_size is no multiple of the heads")
            head_dim = hidden // heads
        eos = raw.get("eos_token_id")
        if eos is None:
            eos_ids: tuple = ()
        elif isinstance(eos, int):
            eos_ids = (eos,)
        else:
            eos_ids = tuple(int(e) for e in eos)
        window = raw.get("sliding_window")
        if not raw.get("use_sliding_window", window is not None):
            window = None
        layers = _positive_int(raw, "num_hidden_layers")
        config = cls(
            vocab_size=_positive_int(raw, "vocab_size"),
            hidden_size=hidden,
            intermediate_size=_positive_int(raw, "intermediate_size"),
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=int(head_dim),
            max_position_embeddings=int(raw.get("max_position_embeddings", 32768)),
            rms_norm_eps=float(_require(raw, "rms_norm_eps")),
            rope_theta=float(_require(raw, "rope_theta")),
            eos_token_ids=eos_ids,
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            attention_bias=bool(raw.get("attention_bias", False)),
            sliding_window=None if window is None else int(window),
            max_window_layers=(
                None if window is None else int(raw.get("max_window_layers", 0))
            ),
        )
        config.validate()
        return config

    @classmethod
    def from_file(cls, path: str | Path) -> "Qwen3Config":
        return cls.from_dict(json.loads(Path(path).read_text()))

    def validate(self) -> None:
        if self.num_attention_heads % self.num_key_value_heads:
            # src/forge_engine/qwen3.py:87-88
            raise ConfigError("num_attention_heads must be a multiple of num_key_value_heads")
        if self.head_dim < 2 or self.head_dim % 2:
            raise ConfigError(f"head_dim={self.head_dim} must be even (rotary pairs)")
        if not (math.isfinite(self.rms_norm_eps) and self.rms_norm_eps > 0):
            raise ConfigError("rms_norm_eps must be positive")
        if not (math.isfinite(self.rope_theta) and self.rope_theta > 0):
            raise ConfigError("rope_theta must be positive")
        if self.sliding_window is not None and self.sliding_window < 1:
            raise ConfigError("sliding_window must be at least 1")
        for eos in self.eos_token_ids:
            if not 0 <= eos < self.vocab_size:
                raise ConfigError(f"eos_token_id {eos} lies outside the vocabulary")

    # -- writing ----------------------------------------------------------------
    def to_dict(self) -> dict:
        eos = list(self.eos_token_ids)
        return {
            "architectures": [self.architecture],
            "model_type": "qwen3",
            "hidden_act": "silu",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "eos_token_id": eos[0] if len(eos) == 1 else (eos or None),
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": self.attention_bias,
            "sliding_window": self.sliding_window,
            "use_sliding_window": self.sliding_window is not None,
            "max_window_layers": self.max_window_layers,
            "torch_dtype": "bfloat16",
        }

    # -- derived ----------------------------------------------------------------
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def layer_window(self, index: int) -> int | None:
        """Layers from ``max_window_layers`` on are windowed when a window is configured."""
        if self.sliding_window is None:
            return None
        return self.sliding_window if index >= (self.max_window_layers or 0) else None

    def to_model_spec(self) -> ModelSpec:
        """Describe the model as parts (formulas: src/forge_engine/qwen3.py:108-261)."""
        layers = []
        for index in range(self.num_hidden_layers):
            prefix = f"model.layers.{index}"
            layers.append(
                LayerSpec(
                    input_norm=NormSpec(self.hidden_size, self.rms_norm_eps),
                    mixer=AttentionSpec(
                        hidden_size=self.hidden_size,
                        num_heads=self.num_attention_heads,
                        num_kv_heads=self.num_key_value_heads,
                        head_dim=self.head_dim,
                        qk_norm=True,
                        qk_norm_eps=self.rms_norm_eps,
                        bias=self.attention_bias,
                        scale=self.head_dim**-0.5,
                        position=RotarySpec(self.head_dim, self.rope_theta, self.head_dim),
                        window=self.layer_window(index),
                    ),
                    post_norm=NormSpec(self.hidden_size, self.rms_norm_eps),
                    ffn=GatedMLPSpec(self.hidden_size, self.intermediate_size, "silu"),
                    names={
                        "input_norm": f"{prefix}.input_layernorm",
                        "mixer": f"{prefix}.self_attn",
                        "post_norm": f"{prefix}.post_attention_layernorm",
                        "ffn": f"{prefix}.mlp",
                    },
                )
            )
        return ModelSpec(
            vocab_size=self.vocab_size,
            hidden_size=self.hidden_size,
            layers=tuple(layers),
            schedule=tuple(RunSpec(i) for i in range(self.num_hidden_layers)),
            final_norm=NormSpec(self.hidden_size, self.rms_norm_eps),
            tie_embeddings=self.tie_word_embeddings,
            max_positions=self.max_position_embeddings,
            eos_token_ids=self.eos_token_ids,
        )

"""Configuration: part specs, the Qwen3 config, engine settings and the registry."""

from .engine import EngineConfig, SchedulerConfig
from .qwen3 import Qwen3Config
from .registry import (
    Architecture,
    architecture_of,
    known_architectures,
    read_model_config,
    register_architecture,
)
from .specs import (
    AttentionSpec,
    GatedMLPSpec,
    LayerSpec,
    ModelSpec,
    NoPositionSpec,
    NormSpec,
    RotarySpec,
    RunSpec,
)

register_architecture(
    Architecture("Qwen3ForCausalLM", Qwen3Config.from_dict, Qwen3Config.to_model_spec),
    replace=True,
)

__all__ = [
    "Architecture",
    "AttentionSpec",
    "EngineConfig",
    "GatedMLPSpec",
    "LayerSpec",
    "ModelSpec",
    "NoPositionSpec",
    "NormSpec",
    "Qwen3Config",
    "RotarySpec",
    "RunSpec",
    "SchedulerConfig",
    "architecture_of",
    "known_architectures",
    "read_model_config",
    "register_architecture",
]

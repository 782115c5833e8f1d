"""forge_engine_b200: a single-GPU Qwen3 inference engine for NVIDIA B200 (sm_100a)."""

__version__ = "0.1.0"

from .config import EngineConfig, Qwen3Config, SchedulerConfig, read_model_config  # noqa: E402,F401
from .errors import (  # noqa: E402,F401
    ConfigError,
    CUDAUnavailableError,
    ForgeEngineError,
    KVCacheCapacityError,
    OverloadedError,
    UnsupportedShapeError,
    WeightsError,
)
from .sampling.params import SamplingParams  # noqa: E402,F401

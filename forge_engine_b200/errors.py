"""Error types raised to users of the engine.

The upstream project has the same three-level idea (src/forge_engine/model.py:18-40):
one base class, a missing-device error and an out-of-memory error.
"""

from __future__ import annotations


class ForgeEngineError(RuntimeError):
    """Base class of every error the engine raises on purpose."""


class ConfigError(ForgeEngineError, ValueError):
    """config.json is missing a key, has a wrong value, or names an unknown architecture."""


class WeightsError(ForgeEngineError):
    """A checkpoint does not match the model: missing, unexpected or misshaped tensors."""


class CUDAUnavailableError(ForgeEngineError):
    """No CUDA device, or the native kernels could not be built or loaded."""


class KVCacheCapacityError(ForgeEngineError):
    """The page pool cannot lease the pages asked for (src/forge_engine/cache.py:14-15)."""


class OverloadedError(ForgeEngineError):
    """Admission refused: the bound on requests is reached or the request can never fit
    (src/forge_engine/scheduler.py:52-53)."""


class UnsupportedShapeError(ForgeEngineError, ValueError):
    """A kernel was asked for a size it does not implement; it refuses instead of guessing."""

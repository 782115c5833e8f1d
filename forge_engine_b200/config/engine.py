"""Engine-level settings: sampling defaults and scheduler limits.

Names and defaults follow upstream (src/forge_engine/config.py:11-37,
src/forge_engine/scheduler.py:56-76); ``chunk_size``, ``dtype`` and ``max_context``
are additions of this engine.
"""

from __future__ import annotations

from dataclasses import dataclass

from ..sampling.params import SamplingParams


@dataclass(frozen=True)
class EngineConfig:
    """Generation defaults of one engine instance."""

    max_new_tokens: int = 256
    temperature: float = 0.0
    top_k: int | None = None
    top_p: float = 1.0
    min_p: float = 0.0
    seed: int | None = None
    dtype: str = "bfloat16"

    def __post_init__(self) -> None:
        self.sampling_params()
        if self.dtype not in ("bfloat16", "float32"):
            raise ValueError("dtype must be 'bfloat16' or 'float32'")

    def sampling_params(self) -> SamplingParams:
        return SamplingParams(
            temperature=self.temperature,
            top_k=self.top_k,
            top_p=self.top_p,
            min_p=self.min_p,
            max_new_tokens=self.max_new_tokens,
            seed=self.seed,
        )


@dataclass(frozen=True)
class SchedulerConfig:
    """Limits of admission and of one scheduling iteration.

    ``block_size`` tokens per page, ``block_capacity`` pages in the pool,
    ``token_budget`` tokens per step over all requests, ``max_batch_size`` requests
    per step, ``max_requests`` admitted and unfinished at once, ``chunk_size`` the
    most prompt tokens of one request in one step (None: only the budget limits it),
    ``lookahead`` lets steps of decoding requests only be launched one ahead of the
    host's bookkeeping (their events then arrive one ``step()`` later).
    """

    max_requests: int = 16
    max_batch_size: int = 8
    token_budget: int = 256
    block_size: int = 16
    block_capacity: int = 1024
    chunk_size: int | None = None
    lookahead: bool = True

    def __post_init__(self) -> None:
        for name in ("max_requests", "max_batch_size", "token_budget", "block_size", "block_capacity"):
            if getattr(self, name) < 1:
                raise ValueError(f"{name} must be at least 1")
        if self.chunk_size is not None and self.chunk_size < 1:
            raise ValueError("chunk_size must be at least 1")

"""Validated sampling parameters (names and rules of src/forge_engine/sampling.py:14-46)."""

from __future__ import annotations

import math
from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    """How the next token is chosen from a row of logits.

    temperature 0 is greedy argmax; otherwise the order is temperature, top-k,
    top-p, min-p, softmax in 32-bit, one draw.  ``seed`` keys the request's own
    random stream; None draws a seed from the engine's generator at admission.
    """

    temperature: float = 0.0
    top_k: int | None = None
    top_p: float = 1.0
    min_p: float = 0.0
    max_new_tokens: int = 256
    seed: int | None = None

    def __post_init__(self) -> None:
        if not math.isfinite(self.temperature) or self.temperature < 0.0:
            raise ValueError("temperature must be finite and non-negative")
        if self.top_k is not None and self.top_k < 1:
            raise ValueError("top_k must be at least 1")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")
        if not 0.0 <= self.min_p <= 1.0:
            raise ValueError("min_p must be in [0, 1]")
        if self.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be at least 1")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0

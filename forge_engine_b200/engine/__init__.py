"""Step function, scheduler and the generation entry point."""

from .batch import StepBatch, StepEntry, build_batch
from .runner import ModelRunner

__all__ = ["ModelRunner", "StepBatch", "StepEntry", "build_batch"]

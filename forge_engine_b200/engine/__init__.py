"""Step function, scheduler and the generation entry point."""

from .batch import StepBatch, StepEntry, build_batch
from .engine import Engine
from .runner import ModelRunner
from .scheduler import RequestStatus, RequestView, Scheduler, SchedulerSnapshot, StreamEvent

__all__ = [
    "Engine",
    "ModelRunner",
    "RequestStatus",
    "RequestView",
    "Scheduler",
    "SchedulerSnapshot",
    "StepBatch",
    "StepEntry",
    "StreamEvent",
    "build_batch",
]

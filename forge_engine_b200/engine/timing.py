"""Device time of the parts of a step, taken with CUDA events.

Upstream times whole operations with CUDA events around them, after warm-up, and reports
minimum, 10th percentile, median, 90th percentile and maximum
(tools/validate_l4.py:136-183).  ``StepTimer`` does the same inside the step function: the
model and its blocks wrap each part's call in ``timer.section(name)``; events are only
recorded, nothing synchronises until ``collect()``.  Timed steps run eagerly (a captured
graph has no places to put events), so the figures include the gaps a launch-bound step has.
"""

from __future__ import annotations

import statistics
from contextlib import contextmanager

import torch


class StepTimer:
    def __init__(self) -> None:
        self._open: list = []      # (name, start event, stop event), not yet read
        self._ms: dict = {}        # name -> list of milliseconds

    @contextmanager
    def section(self, name: str):
        start = torch.cuda.Event(enable_timing=True)
        stop = torch.cuda.Event(enable_timing=True)
        start.record()
        try:
            yield
        finally:
            stop.record()
            self._open.append((name, start, stop))

    def collect(self) -> dict:
        """Synchronise once and return name -> {calls, total_ms, minimum, p10, median, p90,
        maximum} over every section recorded since ``reset()``."""
        if self._open:
            torch.cuda.synchronize()
            for name, start, stop in self._open:
                self._ms.setdefault(name, []).append(float(start.elapsed_time(stop)))
            self._open = []
        out = {}
        for name, values in self._ms.items():
            ordered = sorted(values)
            last = len(ordered) - 1
            out[name] = {
                "calls": len(ordered),
                "total_ms": sum(ordered),
                "minimum": ordered[0],
                "p10": ordered[int(0.10 * last)],
                "median": float(statistics.median(ordered)),
                "p90": ordered[int(0.90 * last)],
                "maximum": ordered[-1],
            }
        return out

    def reset(self) -> None:
        self._open, self._ms = [], {}

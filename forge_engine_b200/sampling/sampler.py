"""Host side of token sampling: packs per-row parameters and launches the kernel.

Upstream samples one request at a time with torch ops and reads each id back with
``.item()`` (src/forge_engine/sampling.py:49-80, src/forge_engine/scheduler.py:472-482).
Here all rows of a step are sampled by one kernel launch and read back by one copy.
"""

from __future__ import annotations

from typing import Sequence

import torch

from ..ops import native
from .params import SamplingParams


def _to_signed64(value: int) -> int:
    value &= (1 << 64) - 1
    return value - (1 << 64) if value >= (1 << 63) else value


class Sampler:
    RING = 4   # pinned result buffers; one is reused four asynchronous calls later

    def __init__(self, device, status: torch.Tensor) -> None:
        self.device = torch.device(device)
        self.status = status
        self._pinned: list = []
        self._turn = 0

    def sample(
        self,
        logits: torch.Tensor,
        params: Sequence[SamplingParams],
        seeds: Sequence[int],
        counters: Sequence[int],
    ) -> torch.Tensor:
        """One token id per row (int32, on the device).  Row i is drawn with
        ``uniform(seeds[i], counters[i])`` unless its temperature is 0 (argmax)."""
        rows = logits.shape[0]
        assert len(params) == rows and len(seeds) == rows and len(counters) == rows
        out = torch.empty(rows, dtype=torch.int32, device=self.device)
        if all(p.greedy for p in params):
            native.sample(logits, out, self.status)
            return out
        floats = torch.tensor(
            [[p.temperature for p in params], [p.top_p for p in params], [p.min_p for p in params]],
            dtype=torch.float32,
        )
        top_k = torch.tensor([p.top_k or 0 for p in params], dtype=torch.int32)
        longs = torch.tensor(
            [[_to_signed64(s) for s in seeds], [_to_signed64(c) for c in counters]], dtype=torch.int64
        )
        floats = floats.pin_memory().to(self.device, non_blocking=True)
        top_k = top_k.pin_memory().to(self.device, non_blocking=True)
        longs = longs.pin_memory().to(self.device, non_blocking=True)
        native.sample(logits, out, self.status, temperature=floats[0], top_k=top_k, top_p=floats[1],
                      min_p=floats[2], seeds=longs[0], counters=longs[1])
        return out

    def sample_to_host(self, logits, params, seeds, counters) -> list:
        return self.sample(logits, params, seeds, counters).tolist()

    def sample_async(self, logits, params, seeds, counters) -> tuple:
        """Sample and start copying the ids to pinned host memory without waiting:
        returns (ids on the device, pinned host tensor, event that marks the copy done)."""
        device = self.sample(logits, params, seeds, counters)
        rows = device.numel()
        # pinned memory is allocated once and reused: allocating it stalls the device
        if not self._pinned or self._pinned[0].numel() < rows:
            self._pinned = [torch.empty(max(rows, 256), dtype=torch.int32).pin_memory() for _ in range(self.RING)]
        host = self._pinned[self._turn % self.RING][:rows]
        self._turn += 1
        host.copy_(device, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return device, host, event

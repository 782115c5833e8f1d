"""CUDA graphs for decode steps.

A decode step at small batch is a few hundred short kernels; issued one by one from
Python they take longer to launch than to run.  Upstream launches everything eagerly and
even synchronises per token (src/forge_engine/engine.py:425).  Here a step in which every
entry brings exactly one token is captured once per *bucket* - (entries rounded up to a
power of two, block-table width rounded up to a power of two) - and replayed: the
step's integers are copied into the graph's fixed device buffer, filler entries pad the
batch to the bucket's size (their keys go to the cache's null page), and the kernels run
with the sizes they were captured with.
"""

from __future__ import annotations

import torch

from ..ops import native
from .batch import BatchPlan, batch_from_buffer, plan_batch


def _bucket(value: int, floor: int = 1) -> int:
    size = floor
    while size < value:
        size *= 2
    return size


class _CapturedStep:
    """One captured graph with its fixed device buffer and a small ring of pinned host
    buffers the step's integers are staged in (a ring, so that a buffer is not rewritten
    while the copy of an earlier step may still be reading it)."""

    RING = 4

    def __init__(self, graph, buffer, logits, launches) -> None:
        self.graph = graph
        self.buffer = buffer
        self.logits = logits
        self.launches = launches
        self.staging = [torch.empty(buffer.numel(), dtype=torch.int32).pin_memory() for _ in range(self.RING)]
        self.views = [t.numpy() for t in self.staging]
        self.events = [None] * self.RING
        self.turn = 0

    def upload(self, flat: list) -> None:
        slot = self.turn % self.RING
        self.turn += 1
        if self.events[slot] is not None:
            self.events[slot].synchronize()
        self.views[slot][:] = flat
        self.buffer.copy_(self.staging[slot], non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self.events[slot] = event


class DecodeGraphs:
    """Captures and replays decode steps of one ModelRunner."""

    def __init__(self, model, cache, max_entries: int) -> None:
        self.model = model
        self.cache = cache
        self.max_entries = max_entries
        self.captured: dict[tuple, _CapturedStep] = {}
        self.pool = None

    def usable(self) -> bool:
        """The model says whether its steps can be captured (it asks its blocks, which ask
        their parts); a model that does not say is run eagerly."""
        return bool(getattr(self.model, "graph_safe", False))

    def _plan(self, entries, bucket_entries: int, width: int, spread: int = 1) -> BatchPlan:
        return plan_batch(entries, self.cache, pad_entries=bucket_entries - len(entries), table_width=width,
                          null_page=self.cache.null_page, null_slot=self.cache.null_slot)

    def _capture(self, key: tuple) -> _CapturedStep:
        bucket_entries, width, spread = key
        device = self.model.ctx.device
        page = self.cache.page_size
        # A batch of filler entries only: it has the bucket's layout and is safe to run.
        plan = self._plan([], bucket_entries, width)
        # The capture sees host-side entries that stand for every step that will be replayed
        # with this graph, so that size decisions made on the host (attention splits) fit
        # them: one entry at the bucket's longest context, the others `spread` times shorter.
        plan.entries = [(0, width * page - 1, 1)] + [(0, max(1, width * page // spread) - 1, 1)] * (bucket_entries - 1)
        plan.max_ctx = width * page
        buffer = torch.tensor(plan.flat, dtype=torch.int32).to(device)
        batch = batch_from_buffer(plan, buffer)
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            for _ in range(2):  # lazy initialisation (handles, attributes) must not be captured
                self.model.forward(batch, self.cache)
        torch.cuda.current_stream(device).wait_stream(side)
        torch.cuda.synchronize(device)
        graph = torch.cuda.CUDAGraph()
        before = native.LAUNCHES
        with torch.cuda.graph(graph, pool=self.pool):
            logits = self.model.forward(batch, self.cache)
        if self.pool is None:
            self.pool = graph.pool()
        return _CapturedStep(graph, buffer, logits, native.LAUNCHES - before)

    def run(self, entries, device_tokens: tuple | None = None) -> torch.Tensor:
        """Replay the step for ``entries`` (one token each; pages already reserved).
        Returns logits for the entries that want them, in entry order.  With
        ``device_tokens = (tensor, rows)`` entry i's token is ``tensor[rows[i]]``, copied
        on the device after the step's other integers have been uploaded."""
        bucket_entries = min(_bucket(len(entries)), _bucket(self.max_entries))
        widest = max(
            (len(self.cache.request(e.key).tables[g].pages) for e in entries for g in range(len(self.cache.groups))),
            default=1,
        )
        # how much longer the longest context is than the average one (a power of two, rounded down)
        pages = [max((len(t.pages) for t in self.cache.request(e.key).tables), default=0) for e in entries]
        spread = 1
        while spread < 32 and widest * len(pages) >= 2 * spread * max(1, sum(pages)):
            spread *= 2
        key = (bucket_entries, _bucket(widest, 8), spread)
        # every entry is laid out as wanting its token, so that the layout is fixed
        wanted = [i for i, e in enumerate(entries) if len(e.want)]
        full = [type(e)(e.key, e.tokens, [0]) for e in entries]
        step = self.captured.get(key)
        if step is None:
            step = self._capture(key)
            self.captured[key] = step
        plan = self._plan(full, *key)
        assert len(plan.flat) == step.buffer.numel()
        step.upload(plan.flat)
        if device_tokens is not None:
            source, rows = device_tokens
            begin, _ = plan.offsets["token_ids"]
            if list(rows) != list(range(len(rows))) or source.numel() != len(rows):
                source = source.index_select(0, torch.tensor(rows, dtype=torch.long, device=source.device))
            step.buffer[begin : begin + len(entries)].copy_(source)
        step.graph.replay()
        native.LAUNCHES += step.launches
        if len(wanted) == len(entries):
            return step.logits[: len(entries)]
        if not wanted:
            return step.logits[:0]
        index = torch.tensor(wanted, dtype=torch.long, device=step.logits.device)
        return step.logits.index_select(0, index)

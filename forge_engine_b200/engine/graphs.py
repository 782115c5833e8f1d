"""CUDA graphs for the steps that are too short to be launched kernel by kernel.

A decode step at small batch is a few hundred short kernels, and so is a step that mixes
a few prompt portions with decoded tokens under a small token budget; issued one by one from
Python they take longer to launch (about 4 ms for 36 layers) than to run.  Upstream launches
everything eagerly and even synchronises per token (src/forge_engine/engine.py:425).  Here a
step is captured once per *bucket* and replayed:

* the bucket fixes the sizes the kernels are launched with: the number of entries (a power
  of two for a decode step, else as it is), the number of tokens (entries for a decode step;
  else a multiple of 32 up to 256, of 64 beyond), the width of the block tables (a power of
  two), and what the model's parts
  decided on the host for this step (``model.plan_step``: for attention, which kernels run and
  with how many splits);
* the step's integers are copied into the graph's fixed device buffer; filler entries pad the
  batch to the bucket's sizes (their tokens sit at positions 0.. of a request that holds only
  the cache's null page, their state is the null slot), and nobody reads their rows;
* every entry is laid out as wanting the logits of its last token, so that the layout does
  not depend on which entries do.

A decode step is captured the first time its bucket is seen.  A bucket of any other step is
captured only when it has been seen ``capture_after`` times (16): a capture takes an eager
pass and the capture itself, up to 0.1 s at 36 layers, and a replay saves a millisecond
or two, so shapes that rarely come back are not worth it (64 requests of 16 to 4,096 tokens
under a budget of 2,048 at the 8B shape: 3.97 s without such captures, 4.4 to 7.2 s when every
bucket seen twice was captured).  Replay would gain even for a 2,048-token prompt (15.3
against 16.2 ms at the 4B shape: the gaps between 330 launches), but steps of more than
``MAX_GRAPH_TOKENS`` tokens (512; FORGE_ENGINE_GRAPH_TOKENS) run eagerly: their shapes vary
too much.  So do steps that want logits elsewhere than at an entry's last token.
"""

from __future__ import annotations

import torch

from ..ops import native
from .batch import BatchPlan, StepEntry, batch_from_buffer, plan_batch

import os

MAX_GRAPH_TOKENS = int(os.environ.get("FORGE_ENGINE_GRAPH_TOKENS", "512"))


def _bucket(value: int, floor: int = 1) -> int:
    size = floor
    while size < value:
        size *= 2
    return size


def _token_bucket(tokens: int) -> int:
    step = 32 if tokens <= 256 else 64
    return -(-tokens // step) * step


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
    """Captures and replays short steps of one ModelRunner."""

    def __init__(self, model, cache, max_entries: int) -> None:
        self.model = model
        self.cache = cache
        self.max_entries = max_entries
        self.captured: dict[tuple, _CapturedStep] = {}
        self.seen: dict[tuple, int] = {}
        self.capture_after = 16       # sightings of a bucket (other than a decode step's) before it is captured
        self.pool = None

    def usable(self) -> bool:
        """The model says whether its steps can be captured (it asks its blocks, which ask
        their parts); a model that does not say is run eagerly."""
        return bool(getattr(self.model, "graph_safe", False))

    def takes(self, entries) -> bool:
        """Whether this step is replayed from a graph: few tokens, and logits wanted at an
        entry's last token or not at all."""
        tokens = 0
        for entry in entries:
            count = len(entry.tokens)
            tokens += count
            want = list(entry.want)
            if want and want != [count - 1]:
                return False
        return tokens == len(entries) or tokens <= MAX_GRAPH_TOKENS

    # -- sizes ---------------------------------------------------------------------
    def _shape(self, entries) -> tuple:
        """(entries, tokens, filler token counts) of the bucket this step runs in."""
        real_entries, real_tokens = len(entries), sum(len(e.tokens) for e in entries)
        if real_tokens == real_entries:                          # one token each: a decode step
            bucket_entries = min(_bucket(real_entries), _bucket(self.max_entries))
            return bucket_entries, bucket_entries, [1] * (bucket_entries - real_entries)
        # tokens go up to the bucket's count; one filler entry takes all the spare ones (none if
        # there are none).  The number of entries is not rounded: every entry adds blocks to the
        # attention kernels' grids, and a step has few.
        bucket_tokens = _token_bucket(real_tokens)
        spare = bucket_tokens - real_tokens
        return real_entries + (1 if spare else 0), bucket_tokens, [spare] if spare else []

    def _plan(self, entries, fillers: list, width: int) -> BatchPlan:
        return plan_batch(entries, self.cache, pad_counts=fillers, table_width=width,
                          null_page=self.cache.null_page, null_slot=self.cache.null_slot)

    def _capture(self, key: tuple, counts: list) -> _CapturedStep:
        """``counts``: tokens per entry of the step that asks for the capture, fillers included
        (any split of the bucket's tokens over its entries has the same layout; this one is known
        to fit block tables of the bucket's width)."""
        bucket_entries, bucket_tokens, width, plans = key
        device = self.model.ctx.device
        # A batch of filler entries only: it has the bucket's layout and is safe to run.
        fillers = list(counts)
        plan = self._plan([], fillers, width)
        assert plan.n_tokens == bucket_tokens and plan.n_entries == bucket_entries
        if bucket_tokens != bucket_entries:
            plan.max_new = bucket_tokens        # no entry brings more; kernels sized by it skip what is not there
        buffer = torch.tensor(plan.flat, dtype=torch.int32).to(device)
        batch = batch_from_buffer(plan, buffer)
        batch.plans = dict(plans)               # what the parts decided on the host for the steps of this bucket
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            # lazy initialisation (handles, function attributes, scratch buffers of this size) must
            # not be captured: one eager pass over the same batch does all of it
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

    def run(self, entries, device_tokens: tuple | None = None) -> torch.Tensor | None:
        """Replay the step for ``entries`` (pages already reserved).  Returns logits for the
        entries that want them, in entry order - or None when the step's bucket has not been
        seen often enough to be captured (the caller then launches it eagerly).  With
        ``device_tokens = (tensor, rows)`` (steps of one token per entry only) entry i's token
        is ``tensor[rows[i]]``, copied on the device after the step's other integers have been
        uploaded."""
        bucket_entries, bucket_tokens, fillers = self._shape(entries)
        widest = max(
            (len(self.cache.request(e.key).tables[g].pages) for e in entries for g in range(len(self.cache.groups))),
            default=1,
        )
        widest = max(widest, -(-max(fillers, default=1) // self.cache.page_size))
        width = _bucket(widest, 8)
        # what the parts decide on the host from the step's real entries (attention: which
        # kernels, how many splits) belongs to the bucket: a graph holds one such decision
        host = [(self.cache.request(e.key).slot, self.cache.request(e.key).length, len(e.tokens)) for e in entries]
        planner = getattr(self.model, "plan_step", None)
        plans = planner(host, self.cache.page_size) if planner is not None else {}
        key = (bucket_entries, bucket_tokens, width, tuple(sorted(plans.items(), key=repr)))
        # every entry is laid out as wanting its last token, so that the layout is fixed
        wanted = [i for i, e in enumerate(entries) if len(e.want)]
        full = [StepEntry(e.key, e.tokens, [len(e.tokens) - 1]) for e in entries]
        step = self.captured.get(key)
        if step is None:
            sightings = self.seen.get(key, 0)
            self.seen[key] = sightings + 1
            if bucket_tokens != bucket_entries and sightings < self.capture_after:
                return None
            step = self._capture(key, [len(e.tokens) for e in entries] + fillers)
            self.captured[key] = step
        plan = self._plan(full, fillers, width)
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
        if wanted == list(range(len(wanted))):          # the first entries want theirs: a view will do
            return step.logits[: len(wanted)]
        index = torch.tensor(wanted, dtype=torch.long, device=step.logits.device)
        return step.logits.index_select(0, index)

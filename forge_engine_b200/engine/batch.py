"""The flat batch one step runs: tokens of several requests side by side.

Upstream has four call shapes - whole prompts of one length, or single tokens of one
cache length, never mixed (src/forge_engine/engine.py:50-279).  Here a step takes any
mix: per entry the request, its next tokens (a portion of a prompt, or one decoded
token) and the places whose logits are wanted.  All integers the kernels need are
packed on the host into one pinned buffer and copied once.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import torch


@dataclass
class StepEntry:
    """``tokens`` are the request's next tokens; ``want`` indexes into them."""

    key: object
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class StepBatch:
    """Device-side description of one step (all tensors int32).

    token_ids, positions, token_entry: [N] - id, absolute position and entry index of
    every token; cu_tokens: [R+1] - where each entry's tokens start; starts, ctx_lens,
    slots: [R] - tokens already cached, tokens after this step, state slot;
    want_rows: [W] - flat token indices whose logits are returned;
    group_tables[g]: [R, P_g] - block table of every entry in layer group g (-1: no page).
    ``entries`` repeats (slot, start, count) on the host for parts written in Python.
    ``shared`` holds what parts work out once per step for all layers (keyed by them).
    """

    n_tokens: int
    n_entries: int
    n_want: int
    token_ids: torch.Tensor
    positions: torch.Tensor
    token_entry: torch.Tensor
    cu_tokens: torch.Tensor
    starts: torch.Tensor
    ctx_lens: torch.Tensor
    slots: torch.Tensor
    want_rows: torch.Tensor
    group_tables: list
    entries: list = field(default_factory=list)
    max_new: int = 0
    max_ctx: int = 0
    shared: dict = field(default_factory=dict)
    # What parts decide on the host for this step, by a key of their own (see
    # ``plan_step`` of the model); filled before a step is captured in a CUDA graph, so that
    # the replayed kernels are the ones the step's real entries call for.
    plans: dict = field(default_factory=dict)


@dataclass
class BatchPlan:
    """The integers of a step laid out in one flat host array, before any copy."""

    flat: list
    offsets: dict          # name -> (begin, length)
    n_tokens: int
    n_entries: int
    n_want: int
    table_widths: list
    entries: list          # (slot, start, count) per entry
    max_new: int
    max_ctx: int


def plan_batch(entries: Sequence[StepEntry], cache, *, pad_counts: Sequence[int] = (), table_width: int | None = None,
               null_page: int | None = None, null_slot: int = 0) -> BatchPlan:
    """Lay out the step's integers.  Pages for the new tokens must already be reserved.

    ``pad_counts`` appends one filler entry per element, with that many tokens at
    positions 0.. of a request that holds only ``null_page`` (a page no request ever holds;
    its keys land there) and whose state slot is ``null_slot`` (a row no request ever
    holds), so that the batch has a fixed number of entries and of tokens; ``table_width``
    fixes the width of every block table.  Both are used by replayed CUDA graphs, whose
    kernels are launched with fixed sizes."""
    token_ids: list[int] = []
    positions: list[int] = []
    token_entry: list[int] = []
    cu = [0]
    starts, ctx_lens, slots, want_rows, host = [], [], [], [], []
    requests = []
    for index, entry in enumerate(entries):
        request = cache.request(entry.key)
        requests.append(request)
        count = len(entry.tokens)
        start = request.length
        token_ids.extend(int(t) for t in entry.tokens)
        positions.extend(range(start, start + count))
        token_entry.extend([index] * count)
        for w in entry.want:
            if not 0 <= w < count:
                raise ValueError(f"request {entry.key!r}: wanted place {w} is outside its {count} tokens")
            want_rows.append(cu[-1] + int(w))
        cu.append(cu[-1] + count)
        starts.append(start)
        ctx_lens.append(start + count)
        slots.append(request.slot)
        host.append((request.slot, start, count))
    pad_entries = len(pad_counts)
    for pad, count in enumerate(pad_counts):
        token_ids.extend([0] * count)
        positions.extend(range(count))
        token_entry.extend([len(entries) + pad] * count)
        want_rows.append(cu[-1] + count - 1)
        cu.append(cu[-1] + count)
        starts.append(0)
        ctx_lens.append(count)
        slots.append(null_slot)
    n, r = cu[-1], len(entries) + pad_entries
    tables = []
    for g in range(len(cache.groups)):
        width = max(1, max((len(req.tables[g].pages) for req in requests), default=1))
        if table_width is not None:
            if width > table_width:
                raise ValueError("a block table is wider than the fixed width")
            width = table_width
        rows = []
        for req in requests:
            pages = req.tables[g].pages
            rows.extend(pages)
            rows.extend([-1] * (width - len(pages)))
        for count in pad_counts:
            pages = -(-count // cache.page_size)
            if pages > width:
                raise ValueError("a filler entry needs a wider block table")
            rows.extend([null_page] * pages)
            rows.extend([-1] * (width - pages))
        tables.append((width, rows))
    flat: list[int] = []
    offsets = {}

    def put(name: str, values: list) -> None:
        offsets[name] = (len(flat), len(values))
        flat.extend(values)
        flat.extend([0] * (-len(flat) % 4))  # keep every array 16-byte aligned

    put("token_ids", token_ids)
    put("positions", positions)
    put("token_entry", token_entry)
    put("cu_tokens", cu)
    put("starts", starts)
    put("ctx_lens", ctx_lens)
    put("slots", slots)
    put("want_rows", want_rows)
    for g, (_, rows) in enumerate(tables):
        put(f"table{g}", rows)
    return BatchPlan(flat, offsets, n, r, len(want_rows), [w for w, _ in tables], host,
                     max([c for _, _, c in host] + list(pad_counts), default=1), max(ctx_lens))


def batch_from_buffer(plan: BatchPlan, device_buffer: torch.Tensor) -> StepBatch:
    """Views of ``device_buffer`` (which holds ``plan.flat``) as a StepBatch."""

    def view(name: str) -> torch.Tensor:
        begin, length = plan.offsets[name]
        return device_buffer[begin : begin + length]

    return StepBatch(
        n_tokens=plan.n_tokens,
        n_entries=plan.n_entries,
        n_want=plan.n_want,
        token_ids=view("token_ids"),
        positions=view("positions"),
        token_entry=view("token_entry"),
        cu_tokens=view("cu_tokens"),
        starts=view("starts"),
        ctx_lens=view("ctx_lens"),
        slots=view("slots"),
        want_rows=view("want_rows"),
        group_tables=[view(f"table{g}").view(plan.n_entries, w) for g, w in enumerate(plan.table_widths)],
        entries=plan.entries,
        max_new=plan.max_new,
        max_ctx=plan.max_ctx,
    )


def upload(flat: list, device) -> torch.Tensor:
    """One pinned host tensor, one asynchronous copy."""
    host_buffer = torch.tensor(flat, dtype=torch.int32)
    if torch.device(device).type == "cuda":
        host_buffer = host_buffer.pin_memory()
    return host_buffer.to(device, non_blocking=True)


def build_batch(entries: Sequence[StepEntry], cache, device) -> StepBatch:
    """Plan, upload and view a step's batch."""
    plan = plan_batch(entries, cache)
    return batch_from_buffer(plan, upload(plan.flat, device))

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


def build_batch(entries: Sequence[StepEntry], cache, device) -> StepBatch:
    """Lay out the step's integers.  Pages for the new tokens must already be reserved."""
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
    n, r = cu[-1], len(entries)
    tables = []
    for g in range(len(cache.groups)):
        width = max(1, max(len(req.tables[g].pages) for req in requests))
        rows = []
        for req in requests:
            pages = req.tables[g].pages
            rows.extend(pages)
            rows.extend([-1] * (width - len(pages)))
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
    host_buffer = torch.tensor(flat, dtype=torch.int32)
    if torch.device(device).type == "cuda":
        host_buffer = host_buffer.pin_memory()
    device_buffer = host_buffer.to(device, non_blocking=True)

    def view(name: str) -> torch.Tensor:
        begin, length = offsets[name]
        return device_buffer[begin : begin + length]

    return StepBatch(
        n_tokens=n,
        n_entries=r,
        n_want=len(want_rows),
        token_ids=view("token_ids"),
        positions=view("positions"),
        token_entry=view("token_entry"),
        cu_tokens=view("cu_tokens"),
        starts=view("starts"),
        ctx_lens=view("ctx_lens"),
        slots=view("slots"),
        want_rows=view("want_rows"),
        group_tables=[view(f"table{g}").view(r, tables[g][0]) for g in range(len(tables))],
        entries=host,
        max_new=max(c for _, _, c in host),
        max_ctx=max(ctx_lens),
    )

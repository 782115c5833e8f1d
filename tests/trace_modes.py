"""Builders of replay traces: the same requests cut in different ways.

Each builder appends steps to a ``Trace`` and records, for every wanted row, which
request and which position it belongs to, so that the caller can compare it with the
plain implementation's whole-sequence logits.
"""

from __future__ import annotations

from dataclasses import dataclass, field


def round_up(value: int, multiple: int) -> int:
    return -(-value // multiple) * multiple


@dataclass
class Trace:
    steps: list = field(default_factory=list)
    rows: list = field(default_factory=list)   # (step, row in step, sequence name, position)
    live: dict = field(default_factory=dict)   # id -> tokens held now
    peak_tokens: int = 0                       # max over time of sum(round_up(held, 64))

    def add_step(self, entries: list, end: tuple = ()) -> None:
        """entries: (request id, sequence name, start, tokens, want)"""
        step = len(self.steps)
        row = 0
        out = []
        for rid, name, start, tokens, want in entries:
            out.append({"id": rid, "tokens": list(tokens), "want": list(want)})
            for w in want:
                self.rows.append((step, row, name, start + w))
                row += 1
            self.live[rid] = self.live.get(rid, 0) + len(tokens)
        assert len(self.live) <= 4, "at most four requests are live at a time"
        self.peak_tokens = max(self.peak_tokens, sum(round_up(n, 64) for n in self.live.values()))
        for rid in end:
            del self.live[rid]
        self.steps.append({"step": step, "entries": out, "end": list(end)})


def whole(trace: Trace, name: str, ids: list) -> None:
    """The request alone, all tokens in one step, logits everywhere."""
    rid = f"whole-{name}"
    trace.add_step([(rid, name, 0, ids, range(len(ids)))], end=(rid,))


def bulk_then_tail(trace: Trace, name: str, ids: list, tail: int = 32) -> None:
    """All but the last ``tail`` tokens in one step, then one token per step."""
    rid = f"tail-{name}"
    tail = min(tail, len(ids) - 1)
    head = len(ids) - tail
    trace.add_step([(rid, name, 0, ids[:head], [head - 1])])
    for i in range(head, len(ids)):
        trace.add_step([(rid, name, i, ids[i : i + 1], [0])], end=(rid,) if i == len(ids) - 1 else ())


def portions(trace: Trace, name: str, ids: list, sizes=(7, 2, 13, 3, 2, 5, 1, 16, 2, 9)) -> None:
    """Portions of changing size, down to two tokens (and one)."""
    rid = f"portions-{name}"
    start, k = 0, 0
    while start < len(ids):
        n = min(sizes[k % len(sizes)], len(ids) - start)
        last = start + n == len(ids)
        trace.add_step([(rid, name, start, ids[start : start + n], range(n))], end=(rid,) if last else ())
        start += n
        k += 1


def mixed(trace: Trace, sequences: dict, prompt_fraction: float = 0.6, chunk=(5, 2, 11, 3)) -> None:
    """Up to four requests live: prompts are fed in portions while others decode one token
    a step; a finished request is ended and the next one starts in its pages."""
    waiting = list(sequences.items())
    live: list = []   # [rid, name, ids, fed, prompt_len]
    tick = 0
    while waiting or live:
        while waiting and len(live) < 4:
            name, ids = waiting.pop(0)
            live.append([f"mixed-{name}", name, ids, 0, max(2, int(len(ids) * prompt_fraction))])
            if len(live) >= 2 and tick == 0:
                break   # let requests join at different times
        entries, ended = [], []
        for slot, item in enumerate(live):
            rid, name, ids, fed, prompt_len = item
            if (tick + slot) % 5 == 4 and fed > 0:
                continue   # this request sits a step out
            if fed < prompt_len:
                n = min(chunk[(tick + slot) % len(chunk)], prompt_len - fed)
                want = [n - 1] if fed + n == prompt_len else ([0] if n > 1 else [])
            else:
                n, want = 1, [0]
            entries.append((rid, name, fed, ids[fed : fed + n], want))
            item[3] = fed + n
            if item[3] == len(ids):
                ended.append(rid)
        if entries:
            trace.add_step(entries, end=tuple(ended))
        live = [item for item in live if item[0] not in ended]
        tick += 1

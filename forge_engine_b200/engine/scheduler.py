"""Continuous, token-budgeted scheduling of many requests over the step function.

States, admission by worst-case page reservation, round-robin order, finishing rules,
cancel and failure clean-up and the observable snapshot follow upstream
(src/forge_engine/scheduler.py:33-553).  Differences, all deliberate:

* prompts are cut into portions: a prompt brings min(what is left of it, chunk_size,
  what is left of the step's token budget) tokens per step, so a step mixes portions of
  prompts with single decoded tokens in one batch (upstream never splits a prompt and
  runs prompts and decodes as separate forwards, scheduler.py:365-411);
* in every step decoding requests take their share of the token budget before prompts;
* a request whose reservation does not fit *now* waits in the queue instead of being
  refused; it is refused (OverloadedError) only if it can never fit or the bound on
  unfinished requests is reached.

When pages run out: they cannot for an admitted request, because admission reserved its
worst case in every layer group.  A waiting request is admitted as soon as finished ones
have returned enough; their pages are then used again.  If the step function still
raises (for instance KVCacheCapacityError from a pool smaller than the scheduler was
told), every request of that step fails and its pages and reservation are returned.
"""

from __future__ import annotations

import random
import time
from collections import deque
from dataclasses import dataclass, field
from enum import Enum
from typing import Sequence

from ..config.engine import SchedulerConfig
from ..errors import OverloadedError
from ..sampling.params import SamplingParams
from .batch import StepEntry


class RequestStatus(str, Enum):
    WAITING = "waiting"      # queued or still feeding its prompt
    RUNNING = "running"      # prompt is in the cache; decoding
    FINISHED = "finished"
    CANCELLED = "cancelled"
    FAILED = "failed"

    @property
    def terminal(self) -> bool:
        return self in (RequestStatus.FINISHED, RequestStatus.CANCELLED, RequestStatus.FAILED)


@dataclass(frozen=True)
class RequestView:
    """Public, immutable state of one request (src/forge_engine/scheduler.py:79-89)."""

    request_id: str
    status: RequestStatus
    prompt_tokens: int
    fed_tokens: int
    sampled_tokens: int
    output_tokens: tuple
    reserved_blocks: tuple
    finish_reason: str | None
    error: str | None


@dataclass(frozen=True)
class StreamEvent:
    """Tokens a request produced in one step, or its change of state."""

    request_id: str
    tokens: tuple
    status: RequestStatus


@dataclass(frozen=True)
class SchedulerSnapshot:
    """Counts for tests and metrics (src/forge_engine/scheduler.py:101-112)."""

    iteration: int
    queued: int
    waiting: int
    running: int
    terminal: int
    reserved_blocks: tuple
    allocated_blocks: tuple
    last_batch: tuple          # (request id, tokens in the step) in batch order
    last_batch_tokens: int
    last_prefill_tokens: int = 0   # of the last step: tokens of prompt portions ...
    last_decode_tokens: int = 0    # ... and decoded tokens fed back (one per decoding request)
    last_step_ms: float = 0.0      # host wall time of the last ``step()`` call
    model_steps: int = 0           # steps that ran the model, and what they ran, since the start
    prefill_tokens: int = 0
    decode_tokens: int = 0
    sampled_tokens: int = 0


@dataclass
class _Inflight:
    """A decode step whose sampled tokens have not been read back yet."""

    requests: list          # row order of the step
    tokens_device: object   # int32 [rows] on the device
    tokens_host: object     # pinned host copy, valid once ``event`` has passed
    event: object


@dataclass
class _Request:
    request_id: str
    prompt: list
    params: SamplingParams
    seed: int
    eos_ids: frozenset
    reservation: list
    status: RequestStatus = RequestStatus.WAITING
    admitted: bool = False
    fed: int = 0
    output: list = field(default_factory=list)
    pending_token: int | None = None
    finish_reason: str | None = None
    error: str | None = None
    reservation_released: bool = False


class Scheduler:
    """``runner`` needs ``.cache`` (a CacheManager) and ``.step(entries) -> logits``;
    ``sampler`` needs ``.sample_to_host(logits, params, seeds, counters) -> list[int]``."""

    def __init__(
        self,
        runner,
        sampler,
        config: SchedulerConfig | None = None,
        default_params: SamplingParams | None = None,
        eos_token_ids: Sequence[int] = (),
        seed: int | None = None,
        vocab_size: int | None = None,
        max_positions: int | None = None,
    ) -> None:
        """``vocab_size`` and ``max_positions`` bound what ``submit`` accepts; left None
        they are read from ``runner.model.spec`` where the runner has a model."""
        self.runner = runner
        self.sampler = sampler
        self.config = config or SchedulerConfig()
        spec = getattr(getattr(runner, "model", None), "spec", None)
        self.vocab_size = vocab_size if vocab_size is not None else getattr(spec, "vocab_size", None)
        self.max_positions = max_positions if max_positions is not None else getattr(spec, "max_positions", None)
        self.default_params = default_params or SamplingParams()
        self.eos_token_ids = frozenset(int(e) for e in eos_token_ids)
        cache = runner.cache
        if cache.page_size != self.config.block_size:
            raise ValueError("cache page size does not match scheduler block_size")
        self._capacity = [g.pool.capacity for g in cache.groups]
        self._reserved = [0] * len(cache.groups)
        self._requests: dict[str, _Request] = {}
        self._queue: deque = deque()   # submitted, not yet admitted (FIFO)
        self._order: deque = deque()   # admitted, unfinished (round-robin)
        self._next_number = 1
        self._iteration = 0
        self._last_batch: tuple = ()
        self._last_split = (0, 0)      # (prompt tokens, decoded tokens) of the last step
        self._last_step_ms = 0.0
        self._totals = {"model_steps": 0, "prefill_tokens": 0, "decode_tokens": 0, "sampled_tokens": 0}
        self._rng = random.Random(seed)
        # Decode steps can be launched one ahead: the next step takes its tokens from the
        # sampler's output on the device while the host is still reading the last ones, so
        # the GPU does not idle during the host's bookkeeping.  Needs a runner that replays
        # captured steps and a sampler that can leave its result on the device.
        self.lookahead = bool(
            self.config.lookahead
            and getattr(runner, "supports_device_tokens", False)
            and hasattr(sampler, "sample_async")
        )
        self._inflight: _Inflight | None = None

    # -- admission -----------------------------------------------------------------
    def _max_portion(self) -> int:
        portion = self.config.token_budget
        if self.config.chunk_size is not None:
            portion = min(portion, self.config.chunk_size)
        return portion

    def submit(
        self,
        prompt: Sequence[int],
        *,
        request_id: str | None = None,
        sampling_params: SamplingParams | None = None,
    ) -> str:
        """Queue a request; refuses only what can never run (src/forge_engine/scheduler.py:199-262)."""
        active = sum(not r.status.terminal for r in self._requests.values())
        if active >= self.config.max_requests:
            raise OverloadedError(f"request limit {self.config.max_requests} is full")
        assigned = self._new_id() if request_id is None else request_id
        if assigned in self._requests:
            raise ValueError(f"duplicate request_id: {assigned}")
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise ValueError("each request must contain one non-empty prompt")
        params = sampling_params or self.default_params
        # What the step function would refuse is refused here, where it costs only this
        # request: inside a step it would fail every request batched with it.
        if self.vocab_size is not None:
            bad = [t for t in prompt if not 0 <= t < self.vocab_size]
            if bad:
                raise ValueError(f"token id {bad[0]} is outside the vocabulary of {self.vocab_size}")
        # the last sampled token is never fed back, so the cache holds prompt + max_new - 1
        if self.max_positions is not None and len(prompt) + params.max_new_tokens - 1 > self.max_positions:
            raise ValueError(
                f"prompt of {len(prompt)} tokens with max_new_tokens={params.max_new_tokens} "
                f"exceeds max_position_embeddings={self.max_positions}"
            )
        reservation = self.runner.cache.worst_case_pages(
            len(prompt) + params.max_new_tokens, self._max_portion()
        )
        for group, (need, capacity) in enumerate(zip(reservation, self._capacity)):
            if need > capacity:
                raise OverloadedError(
                    f"request needs {need} KV blocks in layer group {group} but pool capacity is {capacity}"
                )
        seed = params.seed if params.seed is not None else self._rng.getrandbits(63)
        request = _Request(assigned, prompt, params, seed, self.eos_token_ids, reservation)
        self._requests[assigned] = request
        self._queue.append(assigned)
        return assigned

    def _admit(self) -> None:
        """Move queued requests into the cache while their worst case fits, in FIFO order."""
        while self._queue:
            request = self._requests[self._queue[0]]
            if request.status.terminal:
                self._queue.popleft()
                continue
            fits = all(
                r + need <= cap for r, need, cap in zip(self._reserved, request.reservation, self._capacity)
            )
            if not fits or self.runner.cache.slots.free_count == 0:
                break
            self._queue.popleft()
            self.runner.cache.begin_request(request.request_id)
            for group, need in enumerate(request.reservation):
                self._reserved[group] += need
            request.admitted = True
            self._order.append(request.request_id)

    # -- one iteration -----------------------------------------------------------------
    def _select(self) -> list:
        """Pick the step's requests and token counts.

        The first ``max_batch_size`` unfinished requests in round-robin order are
        visited and then moved to the back of the order, so nobody starves.  Of the
        token budget, decoding requests take their one token each first; what is left
        is dealt to the visited prompts in order, each min(rest of prompt, chunk_size,
        budget left).  A prompt that gets nothing keeps its place at the front.  In the
        batch the decoded tokens stand before the prompt portions."""
        visited = []
        for rid in self._order:
            if len(visited) >= self.config.max_batch_size:
                break
            if not self._requests[rid].status.terminal:
                visited.append(self._requests[rid])
        budget = self.config.token_budget
        decoders = [r for r in visited if r.status is RequestStatus.RUNNING][:budget]
        budget -= len(decoders)
        selected = [(r, 1) for r in decoders]
        for request in visited:
            if request.status is RequestStatus.RUNNING or budget == 0:
                continue
            count = min(len(request.prompt) - request.fed, self._max_portion(), budget)
            selected.append((request, count))
            budget -= count
        for request, _ in selected:
            self._order.remove(request.request_id)
        for request in visited:
            if any(request is chosen for chosen, _ in selected):
                self._order.append(request.request_id)
        return selected

    def step(self) -> list:
        """One scheduling iteration.  With look-ahead, a step of decoding requests only is
        launched before the tokens of the step before it have been read; its events are
        then those of the earlier step."""
        began = time.perf_counter()
        try:
            return self._step()
        finally:
            self._last_step_ms = (time.perf_counter() - began) * 1e3

    def _count(self, prefill: int, decode: int) -> None:
        """Book the tokens of a step that is about to run the model."""
        self._last_split = (prefill, decode)
        self._totals["model_steps"] += 1
        self._totals["prefill_tokens"] += prefill
        self._totals["decode_tokens"] += decode

    def _step(self) -> list:
        if self._inflight is not None:
            if all(r.status.terminal for r in self._inflight.requests):
                self._inflight = None      # everything it decoded for has ended meanwhile
            else:
                return self._step_chained()
        if self.lookahead:
            self._admit()
            decoders = self._all_decoding()
            if decoders:
                return self._launch_ahead(decoders, None)
        return self._step_sync()

    # -- look-ahead ------------------------------------------------------------------
    def _all_decoding(self) -> list:
        """The unfinished requests, if every one of them is decoding and they fit one step."""
        if self._queue:
            return []
        live = [self._requests[rid] for rid in self._order if not self._requests[rid].status.terminal]
        if not live or len(live) > min(self.config.max_batch_size, self.config.token_budget):
            return []
        if any(r.status is not RequestStatus.RUNNING for r in live):
            return []
        return live

    def _launch_ahead(self, requests: list, previous: _Inflight | None) -> list:
        """Launch one decode step for ``requests`` without waiting for its tokens.  With
        ``previous`` the input tokens are that step's sampled ids, still on the device."""
        self._iteration += 1
        self._last_batch = tuple((r.request_id, 1) for r in requests)
        self._count(0, len(requests))
        extra = 0 if previous is None else 1     # tokens sampled but not yet counted on the host
        try:
            if previous is None:
                entries = [StepEntry(r.request_id, [r.pending_token], [0]) for r in requests]
                logits = self.runner.step(entries)
            else:
                rows = [previous.requests.index(r) for r in requests]
                entries = [StepEntry(r.request_id, [0], [0]) for r in requests]
                logits = self.runner.step(entries, device_tokens=(previous.tokens_device, rows))
            device, host, event = self.sampler.sample_async(
                logits,
                [r.params for r in requests],
                [r.seed for r in requests],
                [len(r.output) + extra for r in requests],
            )
        except Exception as error:
            events = []
            for request in requests:
                request.status = RequestStatus.FAILED
                request.finish_reason = "error"
                request.error = f"{type(error).__name__}: {error}"
                self._cleanup(request)
                events.append(StreamEvent(request.request_id, (), request.status))
            self._inflight = None
            self._drop_terminal()
            return events
        self._inflight = _Inflight(list(requests), device, host, event)
        return []

    def _step_chained(self) -> list:
        """Launch the next decode step from the device tokens of the one in flight (if the
        batch can go on unchanged), then read the earlier step's tokens and book them."""
        previous = self._inflight
        self._inflight = None
        events: list[StreamEvent] = []
        live = [r for r in previous.requests if not r.status.terminal]
        # a request whose next token is its last by the length limit does not go on
        survivors = [r for r in live if len(r.output) + 1 < r.params.max_new_tokens]
        others = [self._requests[rid] for rid in self._order
                  if not self._requests[rid].status.terminal and self._requests[rid] not in previous.requests]
        if survivors and not self._queue and not others:
            events.extend(self._launch_ahead(survivors, previous))
        previous.event.synchronize()
        tokens = previous.tokens_host.tolist()
        for request, token in zip(previous.requests, tokens):
            if not request.status.terminal:
                events.extend(self._consume(request, int(token)))
        self._drop_terminal()
        return events

    def _step_sync(self) -> list:
        """Admit, select, run one model step, sample, finish (src/forge_engine/scheduler.py:274-310)."""
        self._admit()
        selected = self._select()
        self._iteration += 1
        self._last_batch = tuple((r.request_id, c) for r, c in selected)
        events: list[StreamEvent] = []
        if not selected:
            self._last_split = (0, 0)
            return events
        decoding = sum(r.status is RequestStatus.RUNNING for r, _ in selected)
        self._count(sum(c for _, c in selected) - decoding, decoding)
        entries, sampling_rows = [], []
        for request, count in selected:
            if request.status is RequestStatus.RUNNING:
                tokens = [request.pending_token]
                wants = True
            else:
                tokens = request.prompt[request.fed : request.fed + count]
                wants = request.fed + count == len(request.prompt)
            entries.append(StepEntry(request.request_id, tokens, [len(tokens) - 1] if wants else []))
            if wants:
                sampling_rows.append(request)
        try:
            logits = self.runner.step(entries)
            sampled = []
            if sampling_rows:
                sampled = self.sampler.sample_to_host(
                    logits,
                    [r.params for r in sampling_rows],
                    [r.seed for r in sampling_rows],
                    [len(r.output) for r in sampling_rows],
                )
        except Exception as error:  # every request of the failed step fails; others go on
            for request, _ in selected:
                request.status = RequestStatus.FAILED
                request.finish_reason = "error"
                request.error = f"{type(error).__name__}: {error}"
                self._cleanup(request)
                events.append(StreamEvent(request.request_id, (), request.status))
            self._drop_terminal()
            return events
        for request, count in selected:
            if request.status is RequestStatus.WAITING:
                request.fed += count
                if request.fed == len(request.prompt):
                    request.status = RequestStatus.RUNNING
        for request, token in zip(sampling_rows, sampled):
            events.extend(self._consume(request, int(token)))
        self._drop_terminal()
        return events

    def _consume(self, request: _Request, token: int) -> list:
        """EOS -> "stop" (the EOS id is counted but not emitted); limit -> "length"
        (src/forge_engine/scheduler.py:472-519)."""
        request.pending_token = token
        self._totals["sampled_tokens"] += 1
        reached_eos = token in request.eos_ids
        emitted: tuple = ()
        if reached_eos:
            sampled = len(request.output) + 1
        else:
            request.output.append(token)
            emitted = (token,)
            sampled = len(request.output)
        if reached_eos or sampled >= request.params.max_new_tokens:
            request.status = RequestStatus.FINISHED
            request.finish_reason = "stop" if reached_eos else "length"
            self._cleanup(request)
        return [StreamEvent(request.request_id, emitted, request.status)]

    def run_until_idle(self) -> list:
        events: list[StreamEvent] = []
        while not self.idle:
            step_events = self.step()
            if not self._last_batch:
                raise RuntimeError("scheduler made no progress")
            events.extend(step_events)
        return events

    # -- lifecycle -----------------------------------------------------------------
    def cancel(self, request_id: str) -> bool:
        request = self._request(request_id)
        if request.status.terminal:
            return False
        request.status = RequestStatus.CANCELLED
        request.finish_reason = "cancelled"
        self._cleanup(request)
        self._drop_terminal()
        return True

    def _cleanup(self, request: _Request) -> None:
        """Return pages, slot and reservation exactly once (src/forge_engine/scheduler.py:521-532)."""
        if request.admitted and self.runner.cache.has_request(request.request_id):
            self.runner.cache.end_request(request.request_id)
        if request.admitted and not request.reservation_released:
            for group, need in enumerate(request.reservation):
                self._reserved[group] -= need
            request.reservation_released = True
        request.pending_token = None

    def _drop_terminal(self) -> None:
        self._order = deque(r for r in self._order if not self._requests[r].status.terminal)
        self._queue = deque(r for r in self._queue if not self._requests[r].status.terminal)

    # -- views ---------------------------------------------------------------------
    @property
    def idle(self) -> bool:
        return all(r.status.terminal for r in self._requests.values())

    def request(self, request_id: str) -> RequestView:
        r = self._request(request_id)
        held = r.admitted and not r.reservation_released
        return RequestView(
            request_id=r.request_id,
            status=r.status,
            prompt_tokens=len(r.prompt),
            fed_tokens=r.fed,
            sampled_tokens=len(r.output) + (1 if r.finish_reason == "stop" else 0),
            output_tokens=tuple(r.output),
            reserved_blocks=tuple(r.reservation) if held else tuple(0 for _ in r.reservation),
            finish_reason=r.finish_reason,
            error=r.error,
        )

    def forget(self, request_id: str) -> None:
        if not self._request(request_id).status.terminal:
            raise ValueError("cannot forget an active request")
        del self._requests[request_id]

    def snapshot(self) -> SchedulerSnapshot:
        requests = list(self._requests.values())
        return SchedulerSnapshot(
            iteration=self._iteration,
            queued=sum(not r.admitted and not r.status.terminal for r in requests),
            waiting=sum(r.admitted and r.status is RequestStatus.WAITING for r in requests),
            running=sum(r.status is RequestStatus.RUNNING for r in requests),
            terminal=sum(r.status.terminal for r in requests),
            reserved_blocks=tuple(self._reserved),
            allocated_blocks=tuple(self.runner.cache.leased_pages()),
            last_batch=self._last_batch,
            last_batch_tokens=sum(c for _, c in self._last_batch),
            last_prefill_tokens=self._last_split[0],
            last_decode_tokens=self._last_split[1],
            last_step_ms=self._last_step_ms,
            **self._totals,
        )

    def _request(self, request_id: str) -> _Request:
        try:
            return self._requests[request_id]
        except KeyError:
            raise KeyError(f"unknown request_id: {request_id}") from None

    def _new_id(self) -> str:
        while True:
            candidate = f"req-{self._next_number}"
            self._next_number += 1
            if candidate not in self._requests:
                return candidate

"""The Python entry point: a model folder (or random weights) in, token ids out.

Upstream's entry points are ``GenerationEngine.from_config(...).stream(messages)`` for
one request (src/forge_engine/engine.py:365-451) and ``ConcurrentGenerationEngine`` with
``submit / step / run_until_idle`` for many (src/forge_engine/scheduler.py:137-320); both
work on chat messages through a tokenizer.  This engine works on token ids: text is the
caller's business.  ``Engine`` offers both manners over one scheduler.
"""

from __future__ import annotations

from pathlib import Path
from typing import Iterator, Sequence

from ..config.engine import EngineConfig, SchedulerConfig
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .runner import ModelRunner
from .scheduler import RequestStatus, Scheduler, StreamEvent


class Engine:
    def __init__(
        self,
        runner: ModelRunner,
        engine_config: EngineConfig | None = None,
        scheduler_config: SchedulerConfig | None = None,
    ) -> None:
        self.runner = runner
        self.engine_config = engine_config or EngineConfig()
        self.scheduler_config = scheduler_config or SchedulerConfig()
        self.sampler = Sampler(runner.ctx.device, runner.ctx.status)
        self.scheduler = Scheduler(
            runner,
            self.sampler,
            self.scheduler_config,
            self.engine_config.sampling_params(),
            eos_token_ids=runner.model.spec.eos_token_ids,
            seed=self.engine_config.seed,
        )

    # -- construction ------------------------------------------------------------------
    @classmethod
    def from_pretrained(
        cls,
        folder: str | Path,
        *,
        engine_config: EngineConfig | None = None,
        scheduler_config: SchedulerConfig | None = None,
        device: str = "cuda:0",
    ) -> "Engine":
        engine_config = engine_config or EngineConfig()
        scheduler_config = scheduler_config or SchedulerConfig()
        runner = ModelRunner.from_folder(
            folder,
            dtype=engine_config.dtype,
            device=device,
            page_size=scheduler_config.block_size,
            num_pages=scheduler_config.block_capacity,
            max_requests=scheduler_config.max_requests,
        )
        return cls(runner, engine_config, scheduler_config)

    @classmethod
    def from_random(
        cls,
        config: dict,
        seed: int,
        *,
        engine_config: EngineConfig | None = None,
        scheduler_config: SchedulerConfig | None = None,
        device: str = "cuda:0",
    ) -> "Engine":
        engine_config = engine_config or EngineConfig()
        scheduler_config = scheduler_config or SchedulerConfig()
        runner = ModelRunner.from_random(
            config,
            seed,
            dtype=engine_config.dtype,
            device=device,
            page_size=scheduler_config.block_size,
            num_pages=scheduler_config.block_capacity,
            max_requests=scheduler_config.max_requests,
        )
        return cls(runner, engine_config, scheduler_config)

    # -- many requests -------------------------------------------------------------------
    def submit(self, prompt: Sequence[int], *, request_id: str | None = None,
               sampling_params: SamplingParams | None = None) -> str:
        return self.scheduler.submit(prompt, request_id=request_id, sampling_params=sampling_params)

    def step(self) -> list:
        return self.scheduler.step()

    def run_until_idle(self) -> list:
        """Step until every request has ended; then read the device status word, so that
        what a kernel flagged (a bad page, a wait that ran out, NaN logits) is raised here."""
        events = self.scheduler.run_until_idle()
        self.runner.check_status()
        return events

    def cancel(self, request_id: str) -> bool:
        return self.scheduler.cancel(request_id)

    def generate(
        self,
        prompts: Sequence[Sequence[int]],
        sampling_params: SamplingParams | Sequence[SamplingParams] | None = None,
    ) -> list:
        """Generate for every prompt (lists of token ids) and return the new ids of each.
        Prompts beyond the scheduler's bounds wait their turn; all run in shared batches."""
        if isinstance(sampling_params, SamplingParams) or sampling_params is None:
            per_prompt = [sampling_params] * len(prompts)
        else:
            per_prompt = list(sampling_params)
            if len(per_prompt) != len(prompts):
                raise ValueError("one SamplingParams per prompt, or one for all")
        pending = list(zip(range(len(prompts)), prompts, per_prompt))
        ids: dict[str, int] = {}
        results: list = [None] * len(prompts)
        while pending or ids:
            while pending:
                active = self.scheduler.snapshot()
                if active.queued + active.waiting + active.running >= self.scheduler_config.max_requests:
                    break
                index, prompt, params = pending.pop(0)
                ids[self.submit(prompt, sampling_params=params)] = index
            self.step()
            for rid in [r for r in ids if self.scheduler.request(r).status.terminal]:
                view = self.scheduler.request(rid)
                if view.status is RequestStatus.FAILED:
                    self.scheduler.forget(rid)
                    raise RuntimeError(f"request {rid} failed: {view.error}")
                results[ids.pop(rid)] = list(view.output_tokens)
                self.scheduler.forget(rid)
        self.runner.check_status()
        return results

    # -- one request, streamed -------------------------------------------------------------
    def stream(self, prompt: Sequence[int], sampling_params: SamplingParams | None = None) -> Iterator[int]:
        """Yield the new token ids of one request as they are sampled; pages are always
        given back, also when the consumer stops early (src/forge_engine/engine.py:449-451)."""
        rid = self.submit(prompt, sampling_params=sampling_params)
        try:
            while not self.scheduler.request(rid).status.terminal:
                for event in self.step():
                    if event.request_id == rid:
                        yield from event.tokens
            view = self.scheduler.request(rid)
            if view.status is RequestStatus.FAILED:
                raise RuntimeError(f"request {rid} failed: {view.error}")
            self.runner.check_status()
        finally:
            self.scheduler.cancel(rid)
            self.scheduler.forget(rid)

"""The step function: model + cache manager + one call that runs a mixed batch.

``ModelRunner.step(entries)`` is the only way tokens reach the model.  The scheduler,
the Python entry point, the command line and the trace-replay tool all call it.
"""

from __future__ import annotations

from pathlib import Path
from typing import Sequence

import torch

from ..cache.manager import CacheManager
from ..config.registry import read_model_config
from ..errors import ForgeEngineError, KVCacheCapacityError
from ..models.decoder import DecoderModel
from ..ops import native
from ..parts.base import BuildContext
from ..weights.loader import open_checkpoint
from ..weights.random_init import RandomTensors
from .batch import StepBatch, StepEntry, build_batch
from .graphs import DecodeGraphs
from .timing import StepTimer

DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "bf16": torch.bfloat16,
          "fp32": torch.float32}


def resolve_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError("dtype must be bfloat16 or float32")
        return name
    try:
        return DTYPES[name]
    except KeyError:
        raise ValueError(f"dtype {name!r} must be 'bfloat16' or 'float32'") from None


class ModelRunner:
    """Owns the model, the cache manager and the device status word."""

    def __init__(self, model: DecoderModel, *, page_size: int, num_pages: int, max_requests: int,
                 use_graphs: bool = True, timing: bool = False) -> None:
        """With ``timing`` every part's call is bracketed by CUDA events (``timings()``
        reads them); timed steps are launched kernel by kernel, never replayed from a graph."""
        self.model = model
        self.ctx = model.ctx
        self.timer = None
        if timing:
            self.timer = self.ctx.timer = StepTimer()
            use_graphs = False
        needs, shares = model.cache_needs()
        self.cache = CacheManager(
            needs,
            page_size=page_size,
            num_pages=num_pages,
            max_requests=max_requests,
            dtype=self.ctx.dtype,
            device=self.ctx.device,
            shares=shares,
        )
        self.steps_run = 0
        self.tokens_run = 0
        self.graphs = DecodeGraphs(model, self.cache, max_requests)
        self.use_graphs = use_graphs and self.graphs.usable()

    # -- construction ------------------------------------------------------------------
    @classmethod
    def from_folder(cls, folder: str | Path, *, dtype="bfloat16", device="cuda:0", page_size: int = 16,
                    num_pages: int = 1024, max_requests: int = 16, use_graphs: bool = True,
                    timing: bool = False) -> "ModelRunner":
        """Model class by config.json's architecture, weights by tensor name."""
        native.require_cuda()
        native.lib()
        engine_dtype = resolve_dtype(dtype)
        arch, _, spec = read_model_config(folder)
        expected = arch.expected_tensors(spec)
        optional = (spec.head_name,) if spec.tie_embeddings else ()
        # tensors reach the device when the model asks for them, layer by layer; what a part
        # fuses (q/k/v rows, gate/up rows) never exists twice for more than one layer
        weights = open_checkpoint(folder, expected, engine_dtype, device, optional)
        return cls.from_tensors(spec, weights, dtype=engine_dtype, device=device, page_size=page_size,
                                num_pages=num_pages, max_requests=max_requests, use_graphs=use_graphs,
                                architecture=arch, timing=timing)

    @classmethod
    def from_random(cls, config: dict, seed: int, *, dtype="bfloat16", device="cuda:0", page_size: int = 16,
                    num_pages: int = 1024, max_requests: int = 16, std: float = 0.02,
                    use_graphs: bool = True, timing: bool = False) -> "ModelRunner":
        """Random weights drawn on the device (benchmark-sized models never touch the disk)."""
        native.require_cuda()
        native.lib()
        engine_dtype = resolve_dtype(dtype)
        arch, _, spec = read_model_config(config)
        weights = RandomTensors(arch.expected_tensors(spec), seed, std=std, dtype=engine_dtype, device=device)
        return cls.from_tensors(spec, weights, dtype=engine_dtype, device=device, page_size=page_size,
                                num_pages=num_pages, max_requests=max_requests, use_graphs=use_graphs,
                                architecture=arch, timing=timing)

    @classmethod
    def from_tensors(cls, spec, weights: dict, *, dtype, device, page_size: int, num_pages: int,
                     max_requests: int, use_graphs: bool = True, architecture=None,
                     timing: bool = False) -> "ModelRunner":
        """``architecture`` (a registry entry) assembles the model; None builds the decoder of
        ``models/decoder.py``."""
        native.require_cuda()
        native.lib()
        status = torch.zeros(1, dtype=torch.int32, device=device)
        ctx = BuildContext(dtype=resolve_dtype(dtype), device=torch.device(device), status=status)
        with torch.cuda.device(ctx.device):
            try:
                model = DecoderModel(spec, weights, ctx) if architecture is None else architecture.build(spec, weights, ctx)
            except BaseException:
                if hasattr(weights, "__exit__"):
                    weights.__exit__(RuntimeError, None, None)
                raise
            if hasattr(weights, "close"):
                weights.close()       # a lazily read checkpoint reports NaN and infinities here
            return cls(model, page_size=page_size, num_pages=num_pages, max_requests=max_requests,
                       use_graphs=use_graphs, timing=timing)

    # -- requests ------------------------------------------------------------------------
    def begin(self, key) -> None:
        self.cache.begin_request(key)

    def end(self, key) -> None:
        self.cache.end_request(key)

    # -- the step ------------------------------------------------------------------------
    @property
    def supports_device_tokens(self) -> bool:
        """Whether ``step`` can take a decode step's input tokens from a device tensor."""
        return self.use_graphs

    def step(self, entries: Sequence[StepEntry], device_tokens: tuple | None = None) -> torch.Tensor:
        """Run the entries' tokens as one batch from the cache earlier steps left.

        ``device_tokens = (int32 tensor on the device, rows)`` replaces the entries' (single)
        tokens by ``tensor[rows[i]]`` without a round trip through the host; only for steps
        in which every entry brings one token, on a runner that replays captured steps.

        Returns 32-bit logits [number of wanted places, vocab] on the device, ordered by
        entry and by ``want``.  Pages are leased before anything runs; if they run out,
        nothing has changed and KVCacheCapacityError is raised."""
        if not entries:
            raise ValueError("a step needs at least one entry")
        keys = [e.key for e in entries]
        if len(set(keys)) != len(keys):
            raise ValueError("a request may appear only once in a step")
        vocab = self.model.spec.vocab_size
        for entry in entries:
            if len(entry.tokens) < 1:
                raise ValueError(f"request {entry.key!r} brings no tokens")
            for token in entry.tokens if device_tokens is None else ():
                if not 0 <= int(token) < vocab:
                    raise ValueError(f"request {entry.key!r}: token id {token} is outside the vocabulary")
            request = self.cache.request(entry.key)
            if request.length + len(entry.tokens) > self.model.spec.max_positions:
                raise ForgeEngineError(
                    f"request {entry.key!r} would exceed max_position_embeddings="
                    f"{self.model.spec.max_positions}"
                )
        reserved = []
        try:
            for entry in entries:
                request = self.cache.request(entry.key)
                self.cache.reserve(entry.key, request.length + len(entry.tokens))
                reserved.append(entry.key)
        except KVCacheCapacityError:
            for key in reserved:
                self.cache.trim(key, self.cache.request(key).length)
            raise
        try:
            with torch.cuda.device(self.ctx.device):
                if device_tokens is not None and not (self.use_graphs and all(len(e.tokens) == 1 for e in entries)):
                    raise ValueError("device tokens need a replayed step of single tokens")
                logits = None
                if self.use_graphs and self.graphs.takes(entries):
                    logits = self.graphs.run(entries, device_tokens)
                    n_tokens = sum(len(e.tokens) for e in entries)
                if logits is None:
                    batch = build_batch(entries, self.cache, self.ctx.device)
                    logits = self.model.forward(batch, self.cache)
                    n_tokens = batch.n_tokens
        except BaseException:
            for key in reserved:
                self.cache.trim(key, self.cache.request(key).length)
            raise
        for entry in entries:
            request = self.cache.request(entry.key)
            self.cache.advance(entry.key, request.length + len(entry.tokens))
        self.steps_run += 1
        self.tokens_run += n_tokens
        return logits

    def timings(self, reset: bool = False) -> dict:
        """Device time per part over the steps run so far (needs ``timing=True``):
        ``{"steps", "tokens", "parts": {name: {calls, total_ms, minimum, p10, median, p90,
        maximum}}}``; "mixer" and "ffn" are whole parts, "mixer.*" what the mixer does inside."""
        if self.timer is None:
            raise ForgeEngineError("this runner was built without timing=True")
        out = {"steps": self.steps_run, "tokens": self.tokens_run, "parts": self.timer.collect()}
        if reset:
            self.timer.reset()
        return out

    def check_status(self) -> None:
        """Read the device status word and the canary words round the cache pools and the
        scratch buffers (synchronises); raise if a kernel flagged anything or wrote beside
        its memory."""
        value = int(self.ctx.status.item())
        damaged = native.damaged_canaries(self.cache.guarded)
        if damaged:
            raise ForgeEngineError("canary words were overwritten beside: " + ", ".join(damaged))
        if value:
            self.ctx.status.zero_()
            reasons = [text for bit, text in native.STATUS_BITS.items() if value & bit]
            raise ForgeEngineError("device status: " + "; ".join(reasons))

"""One registry from an architecture's name to its configuration and model spec.

Upstream has no registry (one pinned checkpoint; docs/architecture.md:67-70 says so);
this is the single place where ``config.json``'s ``architectures[0]`` is looked up.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Callable

from ..errors import ConfigError
from .specs import ModelSpec


@dataclass(frozen=True)
class Architecture:
    """``read(raw_dict) -> config`` and ``spec(config) -> ModelSpec`` of one architecture.

    ``assemble(spec, weights, ctx) -> model`` builds the model from tensors by checkpoint
    name; left None, the decoder of ``models/decoder.py`` is built (embedding, the runs of
    the schedule, final norm, output projection).  An architecture whose data flow differs
    outside the blocks (a scaled embedding, capped logits, a second tower) brings its own:
    any object with ``spec`` (vocab_size, max_positions, eos_token_ids), ``ctx``,
    ``cache_needs() -> (needs per run, shares)`` and ``forward(batch, cache) -> logits``;
    optionally ``graph_safe`` (decode steps may be captured and replayed) and
    ``weight_bytes()``.  ``tensors(spec) -> {checkpoint name: WeightInfo}`` lists what
    ``assemble`` needs; left None, the decoder's list is used.
    """

    name: str
    read: Callable[[dict], object]
    spec: Callable[[object], ModelSpec]
    assemble: Callable | None = None
    tensors: Callable | None = None

    def expected_tensors(self, spec) -> dict:
        if self.tensors is not None:
            return self.tensors(spec)
        from ..models.decoder import expected_tensors

        return expected_tensors(spec)

    def build(self, spec, weights: dict, ctx):
        if self.assemble is not None:
            return self.assemble(spec, weights, ctx)
        from ..models.decoder import DecoderModel

        return DecoderModel(spec, weights, ctx)


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(arch: Architecture, *, replace: bool = False) -> None:
    if arch.name in _ARCHITECTURES and not replace:
        raise ConfigError(f"architecture {arch.name!r} is already registered")
    _ARCHITECTURES[arch.name] = arch


def known_architectures() -> tuple:
    return tuple(sorted(_ARCHITECTURES))


def architecture_of(raw: dict) -> Architecture:
    names = raw.get("architectures") or []
    if isinstance(names, str):
        names = [names]
    if not names:
        raise ConfigError(
            "config.json has no 'architectures' entry; known: " + ", ".join(known_architectures())
        )
    name = names[0]
    if name not in _ARCHITECTURES:
        raise ConfigError(
            f"unknown architecture {name!r}; known: " + ", ".join(known_architectures())
        )
    return _ARCHITECTURES[name]


def read_model_config(source: str | Path | dict) -> tuple:
    """Return ``(architecture, typed config, ModelSpec)`` for a folder, a file or a dict."""
    if isinstance(source, dict):
        raw = source
    else:
        path = Path(source)
        if path.is_dir():
            path = path / "config.json"
        if not path.is_file():
            raise ConfigError(f"no config.json at {path}")
        raw = json.loads(path.read_text())
    arch = architecture_of(raw)
    config = arch.read(raw)
    return arch, config, arch.spec(config)

"""Interfaces of the parts a layer is assembled from, and the registry of their kinds.

A part is built from ``(spec, weights, ctx)``:

* ``spec``    - frozen data with a ``kind`` string (see ``config/specs.py``);
* ``weights`` - dict of the part's own tensors by *local* name (the names of
  ``weight_shapes(spec)``), already on the device;
* ``ctx``     - ``BuildContext``: activation dtype, device, the device status word.

No part knows which model it is in, which layer it is, or what other layers do.

To add a kind: write a spec dataclass with a new ``kind``, a class with the methods of
the matching interface below, and call ``register_part(kind, cls)``.  Nothing else in
the package needs to change; an architecture then names the kind in its LayerSpecs.
"""

from __future__ import annotations

from dataclasses import dataclass

from ..cache.manager import CacheNeeds
from ..errors import ConfigError


class _Nothing:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NOTHING = _Nothing()


@dataclass
class BuildContext:
    """What every part may know about its surroundings."""

    dtype: object  # torch.float32 or torch.bfloat16: dtype of activations and of the KV cache
    device: object
    status: object  # int32[1] device word kernels set error bits in
    timer: object = None  # None, or an object whose ``section(name)`` brackets a part's call with events

    def section(self, name: str):
        """A context manager round one part's work: records events when a timer is set."""
        return _NOTHING if self.timer is None else self.timer.section(name)


@dataclass(frozen=True)
class WeightInfo:
    """Shape and role of one tensor; the role picks the random initialiser."""

    shape: tuple
    role: str = "matrix"  # "matrix" N(0, std) | "norm" 1 + N(0, 0.1) | "bias" N(0, std)


@dataclass
class CacheView:
    """What a mixer sees of the cache for one run.

    ``kv`` is ``(k_cache, v_cache)`` [pages, kv_heads, page_size, head_dim] or None;
    ``group`` indexes ``StepBatch.group_tables``; ``owns`` is False when the run reads
    another run's cache and must not write; ``state`` is [max_requests + 1, *shape] or None
    and is indexed by ``StepBatch.slots`` (the last row belongs to filler entries).
    """

    kv: tuple | None
    group: int | None
    owns: bool
    state: object = None


class Part:
    """Common shape of all parts."""

    # True if the part's work only launches kernels (or capturable torch ops) on the current
    # stream and decides nothing from device data or from the host copy of the entries beyond
    # their counts, so that a decode step can be captured once in a CUDA graph and replayed.
    # A block is replayed only if all of its parts say so; parts defined elsewhere say no
    # unless they set it.
    graph_safe = False

    @classmethod
    def weight_shapes(cls, spec) -> dict:
        """Local tensor name -> WeightInfo."""
        return {}


class Norm(Part):
    """``forward(x) -> y`` and the fused ``add_forward(residual, update) -> y`` which first
    adds ``update`` (may be None) into the 32-bit ``residual`` in place."""

    def forward(self, x):
        raise NotImplementedError

    def add_forward(self, residual, update, row_map=None):
        raise NotImplementedError


class PositionEncoding(Part):
    """Either gives the fused q/k kernel a rotary table (``rotary()`` returns
    ``(inv_freq float32[rotary_dim/2], rotary_dim)``) or returns None there and rewrites
    q and k itself in ``apply(qkv, num_q_heads, num_kv_heads, head_dim, batch)``.  A rotary
    part may also offer ``table(batch)``: cosine and sine of the step's angles
    [tokens, rotary_dim/2, 2], taken once per step and shared by all layers."""

    def rotary(self):
        return None

    def apply(self, qkv, num_q_heads, num_kv_heads, head_dim, batch) -> None:
        return None


class Mixer(Part):
    """Mixes information between the tokens of a request.

    ``cache_needs()`` says what the mixer keeps between steps; ``forward(x, batch,
    cache)`` gets the normalised activations [N, hidden] of all tokens of the step, the
    ``StepBatch`` and its ``CacheView``, and returns the update [N, hidden]."""

    # ``graph_safe`` (see Part): a mixer with state of its own must then index it with the
    # device tensor ``batch.slots`` - filler entries of a replayed batch carry the cache's null
    # slot, a row no request holds - and never with the host copy ``batch.entries``.

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds()

    def forward(self, x, batch, cache: CacheView):
        raise NotImplementedError


class FeedForward(Part):
    """Token-wise ``forward(x) -> update`` [N, hidden]."""

    def forward(self, x):
        raise NotImplementedError


_PARTS: dict[str, type] = {}
_ARRANGEMENTS: dict[str, type] = {}


def register_part(kind: str, cls: type, *, replace: bool = False) -> None:
    if kind in _PARTS and not replace:
        raise ConfigError(f"part kind {kind!r} is already registered")
    _PARTS[kind] = cls


def part_class(spec) -> type:
    kind = getattr(spec, "kind", None)
    if kind not in _PARTS:
        raise ConfigError(f"unknown part kind {kind!r}; known: {', '.join(sorted(_PARTS))}")
    return _PARTS[kind]


def build_part(spec, weights: dict, ctx: BuildContext):
    return part_class(spec)(spec, weights, ctx)


def register_arrangement(name: str, cls: type, *, replace: bool = False) -> None:
    if name in _ARRANGEMENTS and not replace:
        raise ConfigError(f"block arrangement {name!r} is already registered")
    _ARRANGEMENTS[name] = cls


def arrangement_class(name: str) -> type:
    if name not in _ARRANGEMENTS:
        raise ConfigError(
            f"unknown block arrangement {name!r}; known: {', '.join(sorted(_ARRANGEMENTS))}"
        )
    return _ARRANGEMENTS[name]

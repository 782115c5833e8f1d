"""Parts of a layer: norms, position encodings, mixers, feed-forwards, blocks."""

from . import attention, block, ffn, norms, positions  # noqa: F401  (registers the kinds)
from .base import (
    BuildContext,
    CacheView,
    FeedForward,
    Mixer,
    Norm,
    Part,
    PositionEncoding,
    WeightInfo,
    arrangement_class,
    build_part,
    part_class,
    register_arrangement,
    register_part,
)

__all__ = [
    "BuildContext",
    "CacheView",
    "FeedForward",
    "Mixer",
    "Norm",
    "Part",
    "PositionEncoding",
    "WeightInfo",
    "arrangement_class",
    "build_part",
    "part_class",
    "register_arrangement",
    "register_part",
]

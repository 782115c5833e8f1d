"""Paged KV cache management."""

from .manager import CacheManager, CacheNeeds, LayerGroup, PagedKVSpec, RequestCache, StateSpec
from .pages import BlockTable, PagePool, StateSlots

__all__ = [
    "BlockTable",
    "CacheManager",
    "CacheNeeds",
    "LayerGroup",
    "PagePool",
    "PagedKVSpec",
    "RequestCache",
    "StateSlots",
    "StateSpec",
]

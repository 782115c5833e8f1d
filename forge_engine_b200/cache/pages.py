"""Integer page pool, per-request block tables and fixed-size state slots.

Semantics follow upstream's block pool (src/forge_engine/cache.py:145-283): a fixed
capacity, a LIFO free list that hands out ids 0, 1, 2, ... first and reuses the most
recently returned ids first, all-or-nothing leases, and releases that reject ids
that are not leased or are named twice.  Unlike upstream the pool deals in integers
only; the tensors the ids index are owned by ``CacheManager``.
"""

from __future__ import annotations

from ..errors import KVCacheCapacityError


class PagePool:
    """Leases page ids ``0 .. capacity-1``."""

    def __init__(self, capacity: int) -> None:
        if capacity < 1:
            raise ValueError("capacity must be at least 1")
        self._capacity = capacity
        self._free = list(range(capacity - 1, -1, -1))
        self._leased: set[int] = set()

    @property
    def capacity(self) -> int:
        return self._capacity

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def leased_count(self) -> int:
        return len(self._leased)

    def allocate(self, count: int) -> tuple:
        """Lease ``count`` pages or none (src/forge_engine/cache.py:208-234)."""
        if count < 0:
            raise ValueError("allocation count must not be negative")
        if count == 0:
            return ()
        if count > len(self._free):
            raise KVCacheCapacityError(
                f"page pool needs {count} pages but only {len(self._free)} are free"
            )
        taken = tuple(reversed(self._free[-count:]))
        del self._free[-count:]
        self._leased.update(taken)
        return taken

    def release(self, pages) -> None:
        """Give pages back (src/forge_engine/cache.py:236-244)."""
        pages = tuple(pages)
        if len(set(pages)) != len(pages):
            raise ValueError("cannot release a page twice in one call")
        unknown = set(pages) - self._leased
        if unknown:
            raise ValueError(f"cannot release pages that are not leased: {sorted(unknown)}")
        self._leased.difference_update(pages)
        self._free.extend(reversed(pages))

    def is_leased(self, page: int) -> bool:
        return page in self._leased


class BlockTable:
    """Logical page index -> physical page id of one request in one layer group.

    Entries of pages that a window has passed are -1; ``first_live`` is the first
    logical index that still holds a page.
    """

    __slots__ = ("pages", "first_live")

    def __init__(self) -> None:
        self.pages: list[int] = []
        self.first_live = 0

    def live_pages(self) -> list[int]:
        return [p for p in self.pages[self.first_live:] if p >= 0]

    def __len__(self) -> int:
        return len(self.pages)


class StateSlots:
    """Leases slot ids for per-request state of fixed size.

    A slot is leased when a request is admitted and returned with its pages.  The
    Qwen3 mixers keep no such state, so their slot is empty, but the slot id still
    names the request's row in any per-request device table.
    """

    def __init__(self, capacity: int) -> None:
        if capacity < 1:
            raise ValueError("capacity must be at least 1")
        self._capacity = capacity
        self._free = list(range(capacity - 1, -1, -1))
        self._leased: set[int] = set()

    @property
    def capacity(self) -> int:
        return self._capacity

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def leased_count(self) -> int:
        return len(self._leased)

    def lease(self) -> int:
        if not self._free:
            raise KVCacheCapacityError(f"all {self._capacity} request slots are in use")
        slot = self._free.pop()
        self._leased.add(slot)
        return slot

    def release(self, slot: int) -> None:
        if slot not in self._leased:
            raise ValueError(f"slot {slot} is not leased")
        self._leased.remove(slot)
        self._free.append(slot)

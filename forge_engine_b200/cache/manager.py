"""The cache manager: layer groups, pages, block tables and state slots of live requests.

Every *run* of the model's schedule declares what it keeps between steps
(``CacheNeeds``): paged keys and values (all of them, or a window), a fixed-size
state, both or nothing.  Runs with the same paged need form a *layer group*; a group
has a page pool and storage of its own, and each live request has one block table
per group.  Upstream has a single kind of layer, so one block spans all layers
(src/forge_engine/cache.py:39-44, 286-481); its events for giving pages back - a
request finishes, is cancelled or fails (src/forge_engine/scheduler.py:521-532) -
are kept, and one is added: a window has passed a page.

All bookkeeping here is host-side integers; the tensors are only allocated and
handed out.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from ..errors import KVCacheCapacityError
from .pages import BlockTable, PagePool, StateSlots


@dataclass(frozen=True)
class PagedKVSpec:
    """Keys and values of ``num_kv_heads`` heads of ``head_dim``; ``window`` None keeps all."""

    num_kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateSpec:
    """A per-request tensor of fixed ``shape`` (dtype by name, e.g. "float32")."""

    shape: tuple
    dtype: str = "float32"


@dataclass(frozen=True)
class CacheNeeds:
    """What one run keeps between steps."""

    kv: PagedKVSpec | None = None
    state: StateSpec | None = None


@dataclass
class LayerGroup:
    """Runs that share page geometry: one pool, one storage tensor, one table per request."""

    index: int
    spec: PagedKVSpec
    units: list  # run indices that own a cache in this group
    pool: PagePool
    storage: object = None  # [units, 2, pages, kv_heads, page_size, head_dim]

    def unit_slot(self, run: int) -> int:
        return self.units.index(run)


@dataclass
class RequestCache:
    """Everything the cache manager holds for one live request."""

    key: object
    slot: int
    length: int = 0
    tables: list = field(default_factory=list)  # one BlockTable per group


def _ceil_div(a: int, b: int) -> int:
    return -(-a // b)


class CacheManager:
    """Pages, block tables and state slots for up to ``max_requests`` live requests."""

    def __init__(
        self,
        needs: list,
        *,
        page_size: int,
        num_pages: int,
        max_requests: int,
        dtype=None,
        device=None,
        shares: dict | None = None,
    ) -> None:
        """``needs[i]`` is the CacheNeeds of run ``i``; ``shares[i] = j`` lets run ``i``
        read run ``j``'s cache instead of keeping one.  With ``device`` None no tensor
        is allocated (bookkeeping only)."""
        if page_size < 1:
            raise ValueError("page_size must be at least 1")
        self.page_size = page_size
        self.num_pages = num_pages
        self.max_requests = max_requests
        self.dtype = dtype
        self.device = device
        self.shares = dict(shares or {})
        self.null_page = num_pages
        # one state row more than requests can hold: filler entries of fixed-size (replayed)
        # batches read and write it, as their keys go to ``null_page``
        self.null_slot = max_requests
        self.slots = StateSlots(max_requests)
        self.groups: list[LayerGroup] = []
        self._run_group: dict[int, tuple] = {}  # run -> (group index, unit slot)
        self._run_state: dict[int, object] = {}  # run -> state tensor [max_requests, *shape]
        self._state_specs: dict[int, StateSpec] = {}
        self._requests: dict[object, RequestCache] = {}
        self.guarded: list = []          # GuardedBuffers behind the groups' storage (CUDA only)
        by_spec: dict[PagedKVSpec, LayerGroup] = {}
        for run, need in enumerate(needs):
            if run in self.shares:
                continue
            if need is None:
                continue
            if need.kv is not None:
                group = by_spec.get(need.kv)
                if group is None:
                    group = LayerGroup(len(self.groups), need.kv, [], PagePool(num_pages))
                    by_spec[need.kv] = group
                    self.groups.append(group)
                group.units.append(run)
                self._run_group[run] = (group.index, len(group.units) - 1)
            if need.state is not None:
                self._state_specs[run] = need.state
        for run, source in self.shares.items():
            if source not in self._run_group and source not in self._state_specs:
                raise ValueError(f"run {run} shares the cache of run {source}, which keeps none")
            if source in self._run_group:
                self._run_group[run] = self._run_group[source]
        if device is not None:
            self._allocate_storage()

    # -- storage ---------------------------------------------------------------
    def _allocate_storage(self) -> None:
        import torch

        self.guarded = []
        for group in self.groups:
            spec = group.spec
            # one page more than the pool leases: ``null_page`` takes the keys of filler
            # entries of fixed-size (graph-replayed) batches and is never read back
            shape = (len(group.units), 2, self.num_pages + 1, spec.num_kv_heads, self.page_size, spec.head_dim)
            numel = 1
            for extent in shape:
                numel *= extent
            if torch.device(self.device).type == "cuda":
                # canary words before and after the pool: a write to "page -1" or past the
                # last page shows in ``native.damaged_canaries(cache.guarded)``
                from ..ops.native import GuardedBuffer

                buffer = GuardedBuffer(f"cache pool of layer group {group.index}", numel, self.dtype, self.device, zero=True)
                self.guarded.append(buffer)
                group.storage = buffer.data.view(shape)
            else:
                group.storage = torch.zeros(shape, dtype=self.dtype, device=self.device)
        for run, spec in self._state_specs.items():
            self._run_state[run] = torch.zeros(
                (self.max_requests + 1, *spec.shape), dtype=getattr(torch, spec.dtype), device=self.device
            )

    def bytes_per_token(self) -> int:
        """Bytes of keys and values one token occupies over all groups (unwindowed view)."""
        import torch

        size = torch.empty((), dtype=self.dtype).element_size() if self.dtype is not None else 2
        return sum(
            2 * len(g.units) * g.spec.num_kv_heads * g.spec.head_dim * size for g in self.groups
        )

    def group_of_run(self, run: int) -> int | None:
        entry = self._run_group.get(run)
        return None if entry is None else entry[0]

    def kv_of_run(self, run: int) -> tuple:
        """(k_cache, v_cache) tensors [pages, kv_heads, page_size, head_dim] of a run."""
        group_index, unit = self._run_group[run]
        storage = self.groups[group_index].storage
        return storage[unit, 0], storage[unit, 1]

    def view(self, run: int):
        """The CacheView a mixer gets for run ``run``."""
        from ..parts.base import CacheView

        kv = self.kv_of_run(run) if run in self._run_group and self.groups[self._run_group[run][0]].storage is not None else None
        return CacheView(
            kv=kv,
            group=self.group_of_run(run),
            owns=run not in self.shares,
            state=self.state_of_run(run),
        )

    def state_of_run(self, run: int):
        """State tensor [max_requests + 1, *shape] of a run (or of the run it shares with);
        the last row is the null slot of filler entries."""
        return self._run_state.get(self.shares.get(run, run))

    # -- requests ----------------------------------------------------------------
    def has_request(self, key) -> bool:
        return key in self._requests

    def request(self, key) -> RequestCache:
        try:
            return self._requests[key]
        except KeyError:
            raise KeyError(f"unknown request {key!r}") from None

    @property
    def live_requests(self) -> int:
        return len(self._requests)

    def begin_request(self, key) -> RequestCache:
        """Lease a state slot (zeroed) and empty block tables."""
        if key in self._requests:
            raise ValueError(f"request {key!r} is already live")
        slot = self.slots.lease()
        for state in self._run_state.values():
            state[slot].zero_()
        entry = RequestCache(key, slot, 0, [BlockTable() for _ in self.groups])
        self._requests[key] = entry
        return entry

    def pages_for(self, group: LayerGroup, table: BlockTable, new_length: int) -> int:
        """How many more pages ``table`` needs to hold positions below ``new_length``."""
        return max(0, _ceil_div(new_length, self.page_size) - len(table.pages))

    def reserve(self, key, new_length: int) -> None:
        """Lease pages so that positions < new_length exist in every group; all or nothing."""
        entry = self.request(key)
        if new_length < entry.length:
            raise ValueError("a request's length cannot shrink")
        wanted = [self.pages_for(g, t, new_length) for g, t in zip(self.groups, entry.tables)]
        for group, count in zip(self.groups, wanted):
            if count > group.pool.free_count:
                raise KVCacheCapacityError(
                    f"request {key!r} needs {count} more pages in layer group {group.index} "
                    f"but only {group.pool.free_count} are free"
                )
        for group, table, count in zip(self.groups, entry.tables, wanted):
            table.pages.extend(group.pool.allocate(count))

    def trim(self, key, length: int) -> None:
        """Give back pages leased beyond ``length`` (undo of a reserve whose step failed)."""
        entry = self.request(key)
        keep = _ceil_div(max(length, entry.length), self.page_size)
        for group, table in zip(self.groups, entry.tables):
            extra = [p for p in table.pages[keep:] if p >= 0]
            if extra:
                group.pool.release(extra)
            del table.pages[keep:]

    def advance(self, key, new_length: int) -> None:
        """Record that positions < new_length are written; release pages a window has passed."""
        entry = self.request(key)
        if new_length < entry.length:
            raise ValueError("a request's length cannot shrink")
        entry.length = new_length
        for group, table in zip(self.groups, entry.tables):
            window = group.spec.window
            if window is None:
                continue
            # the next query sits at position new_length and sees keys >= new_length - window + 1
            first_needed = new_length - window + 1
            dead_pages = max(0, first_needed) // self.page_size
            dead_pages = min(dead_pages, len(table.pages))
            released = []
            for index in range(table.first_live, dead_pages):
                if table.pages[index] >= 0:
                    released.append(table.pages[index])
                    table.pages[index] = -1
            if released:
                group.pool.release(released)
            table.first_live = max(table.first_live, dead_pages)

    def end_request(self, key) -> None:
        """Give back every page and the slot of a request; afterwards it is unknown."""
        entry = self._requests.pop(key, None)
        if entry is None:
            raise KeyError(f"unknown request {key!r}")
        for group, table in zip(self.groups, entry.tables):
            live = [p for p in table.pages if p >= 0]
            if live:
                group.pool.release(live)
            table.pages.clear()
        self.slots.release(entry.slot)

    # -- accounting ----------------------------------------------------------------
    def worst_case_pages(self, total_length: int, max_portion: int) -> list:
        """Pages per group a request of ``total_length`` tokens can hold at once when it
        is fed at most ``max_portion`` tokens a step."""
        out = []
        full = _ceil_div(total_length, self.page_size)
        for group in self.groups:
            window = group.spec.window
            if window is None:
                out.append(full)
            else:
                span = window - 1 + max_portion  # live keys just before a step's release
                out.append(min(full, _ceil_div(span, self.page_size) + 1))
        return out

    def free_pages(self) -> list:
        return [g.pool.free_count for g in self.groups]

    def leased_pages(self) -> list:
        return [g.pool.leased_count for g in self.groups]

    def check_consistency(self) -> None:
        """Every leased page is held by exactly one live table, and nothing else is leased."""
        for group in self.groups:
            held: list[int] = []
            for entry in self._requests.values():
                held.extend(p for p in entry.tables[group.index].pages if p >= 0)
            if len(held) != len(set(held)):
                raise AssertionError(f"group {group.index}: a page is held twice")
            if set(held) != group.pool._leased:
                raise AssertionError(f"group {group.index}: leased pages and tables disagree")
            if group.pool.free_count + group.pool.leased_count != group.pool.capacity:
                raise AssertionError(f"group {group.index}: a page was lost")
        if self.slots.leased_count != len(self._requests):
            raise AssertionError("slots and live requests disagree")

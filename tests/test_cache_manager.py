"""Page pool, block tables, layer groups, windows and state slots (CPU, integers only)."""

from __future__ import annotations

import random

import pytest

from forge_engine_b200.cache import CacheManager, CacheNeeds, PagedKVSpec, PagePool, StateSlots, StateSpec
from forge_engine_b200.errors import KVCacheCapacityError

FULL = CacheNeeds(kv=PagedKVSpec(2, 16, None))
WINDOWED = CacheNeeds(kv=PagedKVSpec(2, 16, 10))


def test_pool_hands_out_low_ids_first_and_reuses_last_returned_first() -> None:
    pool = PagePool(6)
    assert pool.allocate(3) == (0, 1, 2)
    assert pool.allocate(1) == (3,)
    pool.release((1,))
    pool.release((0,))
    # holes are reused without moving live pages; the first id of the last release comes first
    assert pool.allocate(3) == (0, 1, 4)
    assert pool.free_count == 1 and pool.leased_count == 5


def test_pool_is_transactional_and_checks_releases() -> None:
    pool = PagePool(4)
    pool.allocate(3)
    with pytest.raises(KVCacheCapacityError, match="needs 2 pages but only 1"):
        pool.allocate(2)
    assert pool.free_count == 1
    with pytest.raises(ValueError, match="twice"):
        pool.release((0, 0))
    with pytest.raises(ValueError, match="not leased"):
        pool.release((3,))
    pool.release((0, 1, 2))
    with pytest.raises(ValueError, match="not leased"):
        pool.release((1,))
    assert pool.free_count == 4


def test_slots() -> None:
    slots = StateSlots(2)
    a, b = slots.lease(), slots.lease()
    assert (a, b) == (0, 1)
    with pytest.raises(KVCacheCapacityError):
        slots.lease()
    slots.release(a)
    with pytest.raises(ValueError):
        slots.release(a)
    assert slots.lease() == 0


def test_block_tables_grow_by_whole_pages() -> None:
    cache = CacheManager([FULL, FULL], page_size=4, num_pages=8, max_requests=2)
    assert len(cache.groups) == 1 and cache.groups[0].units == [0, 1]
    cache.begin_request("a")
    cache.reserve("a", 5)
    assert cache.request("a").tables[0].pages == [0, 1]
    cache.advance("a", 5)
    cache.reserve("a", 8)
    assert cache.request("a").tables[0].pages == [0, 1]
    cache.advance("a", 8)
    cache.reserve("a", 9)
    assert cache.request("a").tables[0].pages == [0, 1, 2]
    cache.begin_request("b")
    with pytest.raises(KVCacheCapacityError, match="needs 6 more pages"):
        cache.reserve("b", 24)
    assert cache.request("b").tables[0].pages == [] and cache.free_pages() == [5]
    cache.end_request("a")
    cache.reserve("b", 24)
    # a's pages were returned (2, 1, 0 order reversed -> 0, 1, 2 first)
    assert cache.request("b").tables[0].pages == [0, 1, 2, 3, 4, 5]
    cache.check_consistency()
    cache.end_request("b")
    assert cache.leased_pages() == [0] and cache.slots.leased_count == 0
    with pytest.raises(KeyError):
        cache.end_request("b")


def test_trim_undoes_a_reserve() -> None:
    cache = CacheManager([FULL], page_size=4, num_pages=8, max_requests=2)
    cache.begin_request("a")
    cache.reserve("a", 6)
    cache.advance("a", 6)
    cache.reserve("a", 20)
    assert cache.leased_pages() == [5]
    cache.trim("a", 6)
    assert cache.request("a").tables[0].pages == [0, 1] and cache.leased_pages() == [2]
    cache.check_consistency()


def test_groups_by_need_and_window_release() -> None:
    cache = CacheManager([FULL, WINDOWED, WINDOWED, FULL], page_size=4, num_pages=16, max_requests=2)
    assert [g.units for g in cache.groups] == [[0, 3], [1, 2]]
    assert cache.group_of_run(2) == 1 and cache.group_of_run(3) == 0
    cache.begin_request("a")
    length = 0
    for portion in (7, 6, 1, 1, 9, 2):
        cache.reserve("a", length + portion)
        length += portion
        cache.advance("a", length)
        full, windowed = cache.request("a").tables
        assert all(p >= 0 for p in full.pages) and len(full.pages) == -(-length // 4)
        # window 10: the next query at `length` needs keys >= length - 9
        dead = max(0, length - 9) // 4
        assert windowed.first_live == dead
        assert all(p == -1 for p in windowed.pages[:dead])
        assert all(p >= 0 for p in windowed.pages[dead:])
        cache.check_consistency()
    assert cache.leased_pages()[1] < cache.leased_pages()[0]
    cache.end_request("a")
    assert cache.leased_pages() == [0, 0]


def test_worst_case_pages() -> None:
    cache = CacheManager([FULL, WINDOWED], page_size=4, num_pages=64, max_requests=2)
    full, windowed = cache.worst_case_pages(100, max_portion=8)
    assert full == 25
    assert windowed == -(-(10 - 1 + 8) // 4) + 1
    # simulate: the windowed group never holds more than its worst case
    cache.begin_request("a")
    length, peak = 0, 0
    while length < 100:
        portion = min(8, 100 - length)
        cache.reserve("a", length + portion)
        peak = max(peak, cache.leased_pages()[1])
        length += portion
        cache.advance("a", length)
    assert peak <= windowed


def test_shared_cache_runs_own_no_pages() -> None:
    cache = CacheManager([FULL, FULL, FULL], page_size=4, num_pages=8, max_requests=2, shares={2: 0})
    assert cache.groups[0].units == [0, 1]
    assert cache.group_of_run(2) == 0
    with pytest.raises(ValueError):
        CacheManager([CacheNeeds(), FULL], page_size=4, num_pages=8, max_requests=2, shares={1: 0})


def test_state_slots_are_zeroed_on_lease() -> None:
    import torch

    needs = [CacheNeeds(state=StateSpec((3,), "float32")), FULL]
    cache = CacheManager(needs, page_size=4, num_pages=4, max_requests=2, dtype=torch.float32, device="cpu")
    a = cache.begin_request("a")
    state = cache.state_of_run(0)
    # one row more than requests: the null slot of fixed-size batches' filler entries
    assert state.shape == (3, 3) and cache.null_slot == 2
    state[a.slot] += 5.0
    cache.end_request("a")
    b = cache.begin_request("b")
    assert b.slot == a.slot and float(state[b.slot].abs().sum()) == 0.0
    assert cache.view(0).state is state and cache.view(0).kv is None
    # one page more than the pool leases: the null page of fixed-size batches
    assert cache.view(1).kv[0].shape == (5, 2, 4, 16) and cache.null_page == 4


@pytest.mark.parametrize("seed", range(6))
def test_random_request_orders_lose_no_page(seed: int) -> None:
    """Random begin / grow / end in random order: no page lost, held twice or freed twice."""
    rng = random.Random(seed)
    cache = CacheManager([FULL, WINDOWED, FULL], page_size=4, num_pages=24, max_requests=5)
    live: dict[str, int] = {}
    counter = 0
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and len(live) < 5:
            key = f"r{counter}"
            counter += 1
            cache.begin_request(key)
            live[key] = 0
        elif action < 0.8 and live:
            key = rng.choice(sorted(live))
            portion = rng.choice((1, 1, 1, 2, 3, 7, 16))
            try:
                cache.reserve(key, live[key] + portion)
            except KVCacheCapacityError:
                before = cache.leased_pages()
                cache.check_consistency()
                assert cache.leased_pages() == before
                continue
            if rng.random() < 0.1:  # a step that failed after reserving
                cache.trim(key, live[key])
            else:
                live[key] += portion
                cache.advance(key, live[key])
        elif live:
            key = rng.choice(sorted(live))
            cache.end_request(key)
            del live[key]
        cache.check_consistency()
        for key, length in live.items():
            full = cache.request(key).tables[0]
            assert len(full.pages) >= -(-length // 4)
    for key in list(live):
        cache.end_request(key)
    cache.check_consistency()
    assert cache.leased_pages() == [0, 0] and cache.free_pages() == [24, 24]
    assert cache.slots.free_count == 5

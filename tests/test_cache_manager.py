"""The native page-id pool and the cache manager: no page lost, held twice or freed twice (no GPU)."""

from __future__ import annotations

import random
import threading

import pytest

from distie_b200.cache import BlockPool, CacheExhausted, CacheManager, pages_needed
from distie_b200.parts import CacheNeed, StateNeed

FULL = CacheNeed(num_kv_heads=2, head_dim=16, window=None)
WINDOWED = CacheNeed(num_kv_heads=2, head_dim=16, window=20)


def manager(needs=None, pages=12, page_size=8, seats=4, longest=200, **kw) -> CacheManager:
    needs = needs if needs is not None else {0: FULL, 1: FULL}
    return CacheManager(needs, {}, num_pages=pages, page_size=page_size, max_seats=seats, max_tokens_per_request=longest, **kw)


# -- the native pool (behaviour of core/tests/test_block_pool.cpp:12-86 in the reference) --
def test_pool_hands_out_sequential_ids_and_reuses_last_freed_first():
    pool = BlockPool(6)
    assert list(pool.allocate(3)) == [0, 1, 2]
    pool.free([1])
    pool.free([0])
    assert list(pool.allocate(3)) == [0, 1, 3]
    assert (pool.num_blocks, pool.num_free, pool.num_used) == (6, 2, 4)
    assert abs(pool.utilization - 4 / 6) < 1e-12


def test_pool_is_all_or_nothing():
    pool = BlockPool(4)
    pool.allocate(3)
    with pytest.raises(RuntimeError, match="out of blocks"):
        pool.allocate(2)
    assert pool.num_free == 1
    for bad in ([0, 0], [3], [7], [-1], [0, 9]):
        with pytest.raises(ValueError):
            pool.free(bad)
        assert pool.num_free == 1, "a refused free must change nothing"
    pool.free([0, 1, 2])
    assert pool.num_free == 4
    with pytest.raises(ValueError):
        BlockPool(0)


def test_pool_under_threads():
    pool = BlockPool(64)
    seen, lock = [], threading.Lock()

    def work():
        for _ in range(200):
            try:
                ids = list(pool.allocate(3))
            except RuntimeError:
                continue
            with lock:
                seen.append(tuple(ids))
            pool.free(ids)

    threads = [threading.Thread(target=work) for _ in range(8)]
    [t.start() for t in threads]
    [t.join() for t in threads]
    assert pool.num_free == 64 and seen


def test_pages_needed():
    assert [pages_needed(n, 8) for n in (0, 1, 8, 9, 16)] == [0, 1, 1, 2, 2]
    with pytest.raises(ValueError):
        pages_needed(3, 0)


# -- the manager ---------------------------------------------------------------
def test_layers_with_equal_needs_share_a_group_and_others_do_not():
    cache = manager({0: FULL, 1: WINDOWED, 2: FULL, 3: WINDOWED})
    assert [g.slots for g in cache.groups] == [(0, 2), (1, 3)]
    assert cache.groups[0].pool is not cache.groups[1].pool


def test_grow_is_all_or_nothing_across_groups():
    cache = manager({0: FULL, 1: WINDOWED}, pages=4)
    a, b = cache.open_seat(), cache.open_seat()
    assert cache.grow(a, 24)  # 3 pages in each group
    assert not cache.can_grow(b, 17) and not cache.grow(b, 17)
    assert all(g.pool.num_free == 1 for g in cache.groups), "a refused grow must take nothing"
    assert cache.grow(b, 8)
    assert cache.free_pages() == 0
    cache.close_seat(a)
    assert cache.free_pages() == 3 and cache.free_seats == 3
    with pytest.raises(ValueError):
        cache.close_seat(a)


def test_window_pages_are_given_back_once_passed():
    cache = manager({0: FULL, 1: WINDOWED}, pages=12)
    seat = cache.open_seat()
    cache.grow(seat, 64)
    assert [len(p) for p in cache.pages_held(seat).values()] == [8, 8]
    assert cache.trim(seat, 64) == 5  # keys < 64 - 20 + 1 = 45 are dead: pages 0..4
    held = cache.pages_held(seat)
    assert len(held[0]) == 8 and len(held[1]) == 3
    table = cache.groups[1].host_table[seat]
    assert list(table[:5]) == [-1] * 5 and all(t >= 0 for t in table[5:8])
    cache.grow(seat, 70)  # the next page reuses what the window gave back
    assert len(cache.pages_held(seat)[1]) == 4 and cache.groups[1].pool.num_free == 8
    cache.close_seat(seat)
    assert all(g.pool.num_free == 12 for g in cache.groups)


def test_seats_tables_and_limits():
    cache = manager(pages=30, seats=2, longest=40)
    a, b = cache.open_seat(), cache.open_seat()
    with pytest.raises(CacheExhausted):
        cache.open_seat()
    assert cache.fits_ever(40) and not cache.fits_ever(41)
    with pytest.raises(CacheExhausted):
        cache.grow(a, 41)
    cache.grow(a, 17)
    row = cache.groups[0].host_table[a]
    assert sorted(row[:3]) == sorted(cache.pages_held(a)[0]) and list(row[3:]) == [-1, -1]
    assert list(cache.groups[0].host_table[cache.pad_seat]) == [30] * 5, "the padding seat names the spare page"
    cache.reset_seat(a)
    assert cache.pages_held(a)[0] == [] and cache.free_seats == 0
    cache.close_seat(a)
    cache.close_seat(b)


def test_state_slots_exist_even_when_empty():
    cache = manager()
    assert cache.states == {} and cache.state_slot(0) is None
    with_state = CacheManager({}, {0: StateNeed((3, 2))}, num_pages=1, page_size=8, max_seats=2, max_tokens_per_request=8, device="cpu")
    assert with_state.state_slot(0).shape == (3, 3, 2)
    seat = with_state.open_seat()
    with_state.state_slot(0)[seat] += 1
    with_state.close_seat(seat)
    assert float(with_state.state_slot(0)[with_state.open_seat()].abs().sum()) == 0


@pytest.mark.parametrize("seed", range(5))
def test_random_orders_lose_no_page(seed):
    """Requests grow, are trimmed, reset and closed in random order; the books always balance."""
    rng = random.Random(seed)
    cache = manager({0: FULL, 1: WINDOWED, 2: FULL}, pages=40, page_size=4, seats=6, longest=120)
    live: dict[int, int] = {}
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and cache.free_seats:
            live[cache.open_seat()] = 0
        elif action < 0.7 and live:
            seat = rng.choice(list(live))
            target = min(120, live[seat] + rng.randint(1, 23))
            if cache.grow(seat, target):
                live[seat] = target
                cache.trim(seat, target)
        elif action < 0.8 and live:
            seat = rng.choice(list(live))
            cache.reset_seat(seat)
            live[seat] = 0
        elif live:
            cache.close_seat(live.popitem()[0])
        for group in cache.groups:
            held = [page for seat in live for page in group.pages_of(seat)]
            assert len(held) == len(set(held)), "a page is held twice"
            assert len(held) + group.pool.num_free == group.num_pages, "a page was lost"
            for seat, tokens in live.items():
                pages = group.seats.get(seat)
                first = pages.first if pages else 0
                assert first + len(group.pages_of(seat)) >= pages_needed(tokens, 4)
                assert first <= group.first_needed_page(tokens)
    for seat in list(live):
        cache.close_seat(seat)
    assert all(g.pool.num_free == g.num_pages for g in cache.groups) and cache.free_seats == 6

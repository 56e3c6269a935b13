"""The cache manager: no page lost, held twice or freed twice, under random orders of
requests; windows give pages back early; state slots are handed out and reused (no GPU).
Mirrors the reference's allocator tests (tests/test_scheduler.py:25-116)."""

from __future__ import annotations

import random

import pytest

from mini_gpt_inference_b200.cache import (NO_PAGE, CacheFullError, CacheManager, FixedStateSpec,
                                           PagedKVSpec, PagePool, PoolError)


def _manager(num_pages=8, page_tokens=4, max_requests=4, specs=None):
    specs = specs or [PagedKVSpec(2, 16)] * 3
    return CacheManager(specs, page_tokens, num_pages, max_requests)


def test_pool_hands_out_last_freed_first():
    pool = PagePool(4)
    a = pool.take(3)
    assert a == [0, 1, 2] and pool.num_free == 1
    pool.give_back([1])
    assert pool.take(1) == [1]                         # the page just given back is used again
    pool.check()


def test_pool_refuses_double_free_and_foreign_pages():
    pool = PagePool(4)
    pages = pool.take(2)
    pool.give_back(pages)
    with pytest.raises(PoolError, match="twice"):
        pool.give_back([pages[0]])
    with pytest.raises(PoolError, match="not of this pool"):
        pool.give_back([17])
    with pytest.raises(PoolError, match="asked for"):
        pool.take(5)
    pool.check()


def test_layers_with_equal_needs_share_a_group():
    m = _manager(specs=[PagedKVSpec(2, 16), PagedKVSpec(2, 16, window=8), None, PagedKVSpec(2, 16),
                        FixedStateSpec((4, 4))])
    assert len(m.groups) == 2
    assert m.groups[0].layers == [0, 3] and m.groups[1].layers == [1]
    assert m.state_layers == {4: FixedStateSpec((4, 4))}


def test_reserve_grows_only_at_page_edges_and_is_all_or_nothing():
    m = _manager(num_pages=3, page_tokens=4)
    m.admit("a")
    assert m.reserve("a", 4) and m.num_free_pages() == 2
    m.advance("a", 4)
    assert m.reserve("a", 4) and m.num_free_pages() == 2        # idempotent
    assert m.reserve("a", 5) and m.num_free_pages() == 1        # one more token: one more page
    m.advance("a", 5)
    m.admit("b")
    assert not m.reserve("b", 9)                                # needs 3, one free: nothing taken
    assert m.num_free_pages() == 1 and m.block_table("b", 0) == []
    assert m.can_reserve("b", 4) and not m.can_reserve(None, 5)
    assert m.slot_of("a", 0, 4) == m.block_table("a", 0)[1] * 4
    m.check()


def test_release_gives_everything_back_and_slots_are_reused():
    m = _manager(max_requests=2)
    a, b = m.admit("a"), m.admit("b")
    assert {a.state_slot, b.state_slot} == {0, 1}
    with pytest.raises(CacheFullError):
        m.admit("c")
    m.reserve("a", 10)
    m.release("a")
    assert m.num_free_pages() == 8
    assert m.admit("c").state_slot == a.state_slot              # the freed slot is used again
    with pytest.raises(PoolError):
        m.release("a")                                          # freed twice
    with pytest.raises(PoolError):
        m.admit("c")                                            # admitted twice
    m.check()


def test_advance_past_reserved_pages_is_an_error():
    m = _manager()
    m.admit("a")
    m.reserve("a", 4)
    with pytest.raises(PoolError, match="reserved"):
        m.advance("a", 5)


def test_window_gives_pages_back_early():
    m = CacheManager([PagedKVSpec(1, 16, window=6), PagedKVSpec(1, 16)], page_tokens=4,
                     num_pages=16, max_requests=2)
    m.admit("a")
    for length in range(1, 33):
        assert m.reserve("a", length)
        m.advance("a", length)
        windowed, full = m.block_table("a", 0), m.block_table("a", 1)
        assert NO_PAGE not in full and len(full) == (length + 3) // 4
        # the next query sits at position >= length and reads keys >= length - 5
        first_key = max(0, length - 6 + 1)
        for i, page in enumerate(windowed):
            assert (page == NO_PAGE) == ((i + 1) * 4 <= first_key), (length, i)
        m.check()
    assert m.groups[0].pool.num_used <= 3                       # a window of 6 spans at most 3 pages
    with pytest.raises(PoolError, match="given back"):
        m.slot_of("a", 0, 0)
    m.release("a")
    assert m.groups[0].pool.num_free == 16 and m.groups[1].pool.num_free == 16


def test_every_change_of_a_table_shows_in_its_version():
    """Whoever keeps a copy of a request's tables (the runner's staging buffers do) can tell by
    (serial, version) whether it is stale: a new page, a page a window gave back and a new
    admission under an old name all change it; a token inside a page does not."""
    m = _manager(num_pages=8, page_tokens=4, specs=[PagedKVSpec(2, 16, window=6)])
    a = m.admit("a")
    seen = [(a.serial, a.version, [list(t) for t in a.tables])]
    for length in range(1, 21):
        assert m.reserve("a", length)
        m.advance("a", length)
        now = (a.serial, a.version, [list(t) for t in a.tables])
        assert (now[:2] == seen[-1][:2]) == (now[2] == seen[-1][2]), f"length {length}"
        seen.append(now)
    assert len({s[:2] for s in seen}) > 5                       # pages came and went
    m.release("a")
    again = m.admit("a")
    assert again.serial != a.serial


def test_groups_have_page_geometries_of_their_own():
    """A group takes the manager's page size and pool unless its spec names others; a windowed
    group is sized for what its requests can hold at once when the step size is known."""
    specs = [PagedKVSpec(2, 16), PagedKVSpec(2, 16, page_tokens=16), PagedKVSpec(2, 16, window=10),
             PagedKVSpec(1, 8, page_tokens=2, num_pages=7)]
    m = CacheManager(specs, page_tokens=4, num_pages=32, max_requests=3, window_slack_tokens=6)
    # default; same tokens in larger pages; window 10 + 6 per step -> 4 + 2 pages per request slot; as named
    assert [(g.page_tokens, g.num_pages) for g in m.groups] == [(4, 32), (16, 8), (4, 18), (2, 7)]
    assert [m.max_pages_per_request(40, g) for g in range(4)] == [10, 3, 10, 20]
    m.admit("a")
    assert m.pages_needed("a", 13) == [4, 1, 4, 7]
    assert m.tokens_that_fit("a") == 14                          # the smallest pool decides: 7 pages of 2
    assert m.reserve("a", 13) and m.get("a").capacity == 14
    m.advance("a", 13)
    assert not m.reserve("a", 15) and m.get("a").capacity == 14  # group 3 is full: nothing was taken anywhere
    assert [len(t) for t in m.get("a").tables] == [4, 1, 4, 7]
    assert m.slot_of("a", 1, 13 - 1) == m.block_table("a", 1)[0] * 16 + 12
    assert m.slot_of("a", 3, 5) == m.block_table("a", 3)[2] * 2 + 1
    assert m.can_ever_hold(14) and not m.can_ever_hold(15)
    m.check()
    m.release("a")
    assert all(g.pool.num_free == g.num_pages for g in m.groups)
    # without a known step size a windowed group keeps the default pool
    assert CacheManager(specs[2:3], 4, 32, 3).groups[0].num_pages == 32


@pytest.mark.parametrize("mixed", [False, True])
def test_random_orders_lose_nothing(mixed):
    rng = random.Random(0)
    specs = [PagedKVSpec(2, 8), PagedKVSpec(2, 8, window=10), FixedStateSpec((3,))]
    if mixed:
        specs += [PagedKVSpec(2, 8, page_tokens=8, num_pages=14), PagedKVSpec(1, 8, window=5, page_tokens=2)]
    m = CacheManager(specs, page_tokens=4, num_pages=24, max_requests=5)
    live: dict[str, int] = {}
    counter = 0
    for _ in range(3000):
        action = rng.random()
        if action < 0.25 and len(live) < 5:
            rid = f"r{counter}"
            counter += 1
            m.admit(rid)
            live[rid] = 0
        elif action < 0.8 and live:
            rid = rng.choice(list(live))
            new_len = live[rid] + rng.choice([1, 1, 1, 2, 5, 13])
            if m.reserve(rid, new_len):
                m.advance(rid, new_len)
                live[rid] = new_len
            else:
                victim = rng.choice(list(live))                 # make room like a preemption
                m.release(victim)
                del live[victim]
        elif live:
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
        m.check()
        assert m.stats()["live_requests"] == len(live)
    for rid in list(live):
        m.release(rid)
    m.check()
    assert all(g.pool.num_free == g.num_pages for g in m.groups) and m.slots.num_free == 5
    assert [g.num_pages for g in m.groups] == ([24, 24, 14, 48] if mixed else [24, 24])
    assert m.stats()["internal_fragmentation_slots"] == 0


def test_fragmentation_stats():
    # as src/minigpt_infer/cache/paged.py:83-94: slots allocated but unused in tail pages
    m = _manager(num_pages=8, page_tokens=4, specs=[PagedKVSpec(1, 8)])
    m.admit("a")
    m.reserve("a", 5)
    m.advance("a", 5)
    s = m.stats()
    assert s["free_blocks"] == 6 and s["allocated_blocks"] == 2
    assert s["internal_fragmentation_slots"] == 3

"""The cache manager on the CPU: no page lost, held twice or freed twice, under random
orders of requests; windowed groups give pages back as the window passes; rows are reused."""

from __future__ import annotations

import random

import pytest

from ayaka_b200.cache.manager import CacheManager, PagePool
from ayaka_b200.cache.storage import plan_cache
from ayaka_b200.errors import CapacityError, ConfigError, EngineError
from ayaka_b200.parts.base import CacheNeed, StateNeed
from ayaka_b200.parts.spec import Run

FULL = CacheNeed(4, 16, 0)
WINDOW = CacheNeed(2, 32, 40)


def manager(needs=(FULL,), pages=9, page_size=16, requests=3, width=8):
    return CacheManager(list(needs), [pages] * len(needs), page_size, requests, width)


def test_pool_hands_out_each_page_once_and_reuses_freed_pages_first():
    pool = PagePool(5)
    taken = [pool.take() for _ in range(4)]
    assert taken == [1, 2, 3, 4] and pool.take() is None
    pool.give(2)
    pool.give(4)
    assert pool.take() == 4 and pool.take() == 2  # last freed first
    with pytest.raises(EngineError):
        pool.give(0)
    pool.give(3)
    with pytest.raises(EngineError):
        pool.give(3)  # freed twice
    with pytest.raises(CapacityError):
        PagePool(1)


def test_allocate_commit_free():
    m = manager()
    assert m.allocate("a", 17) and m.row("a") == 0
    assert m.tables[0][0, :3].tolist() == [1, 2, 0]
    assert m.allocate("a", 17) and m.num_free_pages() == 6  # idempotent before commit
    m.commit("a", 17)
    assert m.committed("a") == 17
    assert m.allocate("a", 1) and m.num_free_pages() == 6  # slot 17 lies in page 2
    m.commit("a", 1)
    assert m.allocate("a", 15) and m.num_free_pages() == 5
    with pytest.raises(EngineError):
        m.commit("a", 16)  # more than allocated
    m.commit("a", 15)
    m.check_integrity()
    assert m.allocate("b", 1) and m.row("b") == 1
    m.free("a")
    m.free("a")  # unknown id: ignored
    assert m.num_free_pages() == 7 and m.tables[0][0].tolist() == [0] * 8
    assert m.allocate("c", 1) and m.row("c") == 0  # the freed row is reused first
    assert m.tables[0][0, 0] == 1  # and so are the freed pages, in ascending order
    m.check_integrity()


def test_allocate_says_no_without_side_effects():
    m = manager(pages=4, requests=2, width=2)  # 3 usable pages, 32 tokens per request
    assert not m.allocate("a", 33)  # wider than the table row
    assert "a" not in m and m.num_free_pages() == 3
    assert m.allocate("a", 32)
    assert not m.allocate("b", 17)  # two pages wanted, one free
    assert "b" not in m
    assert m.allocate("b", 16)
    assert not m.allocate("c", 1)  # no row left
    m.check_integrity()
    assert m.max_tokens_per_request == 32 and m.max_context_tokens == 32
    assert m.take_fresh_rows() == [0, 1] and m.take_fresh_rows() == []


def test_window_group_gives_pages_back_as_the_window_passes():
    m = manager(needs=(FULL, WINDOW), pages=12, width=10)
    assert m.allocate("a", 100)
    m.commit("a", 100)
    # the next row (position 100) sees keys 61..100: pages 0..2 of the windowed group are gone
    assert m.tables[1][0, :8].tolist()[:3] == [0, 0, 0]
    assert all(m.tables[1][0, 3:7] != 0)
    assert all(m.tables[0][0, :7] != 0)  # the full group keeps everything
    assert m.num_free_pages(0) == 11 - 7 and m.num_free_pages(1) == 11 - 4
    m.check_integrity()
    for _ in range(40):
        assert m.allocate("a", 1)
        m.commit("a", 1)
        m.check_integrity()
    assert m.num_free_pages(1) >= 11 - 4  # never holds more than window / page + 2 pages
    # all groups or none: the full group is exhausted first
    assert not m.allocate("b", 16 * 3)
    assert "b" not in m and m.num_free_pages(1) >= 7
    m.free("a")
    assert m.num_free_pages(0) == 11 and m.num_free_pages(1) == 11
    m.check_integrity()


def test_integrity_check_sees_corruption():
    m = manager()
    m.allocate("a", 40)
    m.commit("a", 40)
    m.tables[0][0, 1] = 0  # a page is lost
    with pytest.raises(EngineError):
        m.check_integrity()
    m = manager()
    m.allocate("a", 20)
    m.allocate("b", 20)
    m.tables[0][1, 0] = m.tables[0][0, 0]  # held twice
    with pytest.raises(EngineError):
        m.check_integrity()
    m = manager()
    m.allocate("a", 20)
    m.pools[0].give(int(m.tables[0][0, 0]))  # both free and held
    with pytest.raises(EngineError):
        m.check_integrity()


@pytest.mark.parametrize("seed", range(12))
def test_random_orders_of_requests_never_lose_a_page(seed):
    rng = random.Random(seed)
    needs = (FULL, WINDOW) if seed % 2 else (FULL,)
    m = manager(needs=needs, pages=rng.randint(6, 20), page_size=rng.choice([4, 16]),
                requests=rng.randint(1, 5), width=rng.randint(4, 12))
    live: dict[str, int] = {}
    counter = 0
    for _ in range(400):
        action = rng.random()
        if action < 0.45 and live:
            rid = rng.choice(list(live))
            n = rng.randint(1, 3 * m.page_size)
            before = [m.num_free_pages(g) for g in range(len(needs))]
            if m.allocate(rid, n):
                done = rng.randint(0, n)
                m.commit(rid, done)
                live[rid] += done
                assert m.committed(rid) == live[rid]
            else:
                assert [m.num_free_pages(g) for g in range(len(needs))] == before
        elif action < 0.75:
            counter += 1
            rid = f"r{counter}"
            n = rng.randint(0, 2 * m.page_size)
            if m.allocate(rid, n):
                m.commit(rid, n)
                live[rid] = n
            else:
                assert rid not in m
        elif live:
            rid = rng.choice(list(live))
            m.free(rid)
            del live[rid]
        m.check_integrity()
        assert sorted(m.live_requests()) == sorted(live)
    for rid in list(live):
        m.free(rid)
    m.check_integrity()
    for group, pool in enumerate(m.pools):
        assert m.num_free_pages(group) == pool.num_usable


def test_plan_groups_runs_by_need_and_shares_read_caches():
    order = (Run(0), Run(1), Run(0), Run(2, reads_cache_of=1), Run(3))
    needs = [(FULL, None), (WINDOW, None), (FULL, None), (WINDOW, None),
             (None, StateNeed((8, 4)))]
    plan = plan_cache(order, needs)
    assert plan.groups == (FULL, WINDOW)
    assert plan.run_group == (0, 1, 0, 1, None)
    assert plan.run_slot == (0, 0, 1, 0, None)  # layer 0 runs twice: two slots; run 3 shares
    assert plan.run_writes == (True, True, True, False, False)
    assert plan.slots_per_group == (2, 1)
    assert plan.run_state[4] == StateNeed((8, 4)) and plan.run_state[0] is None
    assert plan.bytes_per_page(0, 2, 16) == 2 * 2 * 4 * 16 * 16 * 2
    with pytest.raises(ConfigError):
        plan_cache((Run(0), Run(1, reads_cache_of=0)), [(FULL, None), (WINDOW, None)])

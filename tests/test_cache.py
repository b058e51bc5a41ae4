"""The cache manager on the host: no page is lost, held twice or freed twice; windows give pages back;
steps reserve all or nothing; random orders of requests."""
import random

import pytest
import torch

from vitna_anchor_b200.cache import (CacheError, CacheManager, KVSpec, OutOfPages, PageGroup, PagePool, PageTables,
                                     SlotPool, StateSpec, UNMAPPED)


def test_pool_alloc_free_reuse():
    pool = PagePool(3)
    a, b, c = pool.alloc("x"), pool.alloc("x"), pool.alloc("y")
    assert sorted([a, b, c]) == [0, 1, 2] and pool.free_pages == 0
    with pytest.raises(OutOfPages):
        pool.alloc("z")
    pool.free(b, "x")
    assert pool.alloc("z") == b                    # the page just given back is the next one used
    with pytest.raises(CacheError):
        pool.free(a, "y")                          # a foreign page
    pool.free(a, "x")
    with pytest.raises(CacheError):
        pool.free(a, "x")                          # freed twice
    with pytest.raises(CacheError):
        pool.free(17, "x")
    pool.check()


def test_slots_lowest_first():
    s = SlotPool(3)
    assert [s.acquire("a"), s.acquire("b"), s.acquire("c")] == [0, 1, 2]
    with pytest.raises(CacheError):
        s.acquire("d")
    s.release(1, "b")
    with pytest.raises(CacheError):
        s.release(1, "b")
    assert s.acquire("e") == 1


def _tables(pages=8, page_size=4, window=0, max_requests=4):
    return PageTables([PageGroup((0, 1), 2, 16, window)], page_size, [pages], max_requests)


def test_reserve_commit_rollback_close():
    t = _tables()
    t.open("a")
    t.reserve("a", 5)                              # positions 0..4: two pages
    assert t.pools[0].free_pages == 6 and t.get("a").reserved == 5
    t.rollback("a")
    assert t.pools[0].free_pages == 8 and t.get("a").length == 0
    t.reserve("a", 5); t.commit("a")
    assert t.get("a").length == 5
    t.reserve("a", 3); t.commit("a")               # 5..7 fit the second page
    assert t.pools[0].free_pages == 6
    t.reserve("a", 1)                              # position 8: a third page
    assert t.pools[0].free_pages == 5
    t.rollback("a")
    assert t.pools[0].free_pages == 6 and t.get("a").length == 8
    assert t.slot_of_position("a", 0, 5) == t.get("a").tables[0].blocks[1] * 4 + 1
    t.check()
    t.close("a")
    assert t.pools[0].free_pages == 8
    with pytest.raises(CacheError):
        t.close("a")
    t.check()


def test_out_of_pages_changes_nothing():
    t = _tables(pages=3)
    t.open("a"); t.open("b")
    t.reserve("a", 8); t.commit("a")
    before = (t.pools[0].free_pages, list(t.get("b").tables[0].blocks))
    with pytest.raises(OutOfPages):
        t.reserve("b", 5)
    assert (t.pools[0].free_pages, list(t.get("b").tables[0].blocks)) == before
    assert not t.can_reserve([("b", 5)]) and t.can_reserve([("b", 4)])
    assert not t.can_reserve([("a", 1), ("b", 4)])     # together they need two pages, one is free
    t.check()


def test_truncate():
    t = _tables()
    t.open("a"); t.reserve("a", 14); t.commit("a")
    assert t.pools[0].free_pages == 4
    t.truncate("a", 9)
    assert t.get("a").length == 9 and t.pools[0].free_pages == 5
    t.truncate("a", 0)
    assert t.pools[0].free_pages == 8
    with pytest.raises(CacheError):
        t.truncate("a", 3)
    t.check()


def test_window_gives_pages_back():
    t = _tables(pages=6, page_size=4, window=6)
    t.open("a")
    for _ in range(40):                             # far more positions than the pool holds
        t.reserve("a", 1); t.commit("a")
        t.check()
    blocks = t.get("a").tables[0].blocks
    assert len(blocks) == 10 and blocks[:8] == [UNMAPPED] * 8      # next query at 40 needs keys from 35: block 8 on
    assert t.pools[0].free_pages == 4
    with pytest.raises(CacheError):
        t.truncate("a", 20)                         # those pages are gone
    t.close("a"); t.check()
    assert t.pools[0].free_pages == 6


def test_manager_groups_by_need_and_state_slots():
    specs = [KVSpec(2, 16), KVSpec(2, 16, window=8), KVSpec(2, 16), StateSpec((3, 5)), None]
    m = CacheManager(specs, page_size=4, num_pages=[10, 4], max_requests=2, dtype=torch.float32, device="cpu")
    assert [g.cache_ids for g in m.groups] == [(0, 2), (1,)]
    assert m.pools[0].shape == (2, 10, 2, 2, 4, 16) and m.pools[1].shape == (1, 4, 2, 2, 4, 16)
    assert m.views[3].state.shape == (2, 3, 5) and m.views[4].pages is None and m.views[4].state is None
    assert m.views[2].pages.data_ptr() == m.pools[0][1].data_ptr()
    slot = m.open("r")
    m.views[3].state[slot] += 1
    with pytest.raises(OutOfPages):
        m.reserve_step([("r", 30)])                 # a portion needs pages for all of its positions, in the window group too
    for _ in range(6):
        m.reserve_step([("r", 5)]); m.commit_step([("r", 5)])
    assert m.free_pages() == [2, 1]                 # all 8 pages of the full group; the window kept 3 of 8
    m.close("r")
    assert m.open("s") == slot and float(m.views[3].state[slot].abs().sum()) == 0.0     # a slot starts at zero
    with pytest.raises(OutOfPages):
        m.reserve_step([("s", 41)])
    assert m.free_pages() == [10, 4]
    m.check()


@pytest.mark.parametrize("seed", range(5))
def test_random_orders_keep_every_page_accounted(seed):
    rng = random.Random(seed)
    t = PageTables([PageGroup((0,), 1, 16, 0), PageGroup((1,), 1, 16, 7)], 4, [24, 9], 5)
    live, n = {}, 0
    for _ in range(600):
        r = rng.random()
        if r < 0.15 and len(live) < 5:
            n += 1
            t.open(n); live[n] = 0
        elif r < 0.75 and live:
            rid = rng.choice(list(live))
            k = rng.randint(1, 9)
            try:
                t.reserve(rid, k)
            except OutOfPages:
                pass
            else:
                if rng.random() < 0.15:
                    t.rollback(rid)
                else:
                    t.commit(rid); live[rid] += k
        elif r < 0.85 and live:
            rid = rng.choice(list(live))
            try:
                cut = rng.randint(0, live[rid])
                t.truncate(rid, cut); live[rid] = cut
            except CacheError:
                pass                                # behind the window
        elif live:
            rid = rng.choice(list(live))
            t.close(rid); del live[rid]
        t.check()
        for rid, length in live.items():
            assert t.get(rid).length == length
    for rid in list(live):
        t.close(rid)
    t.check()
    assert [p.free_pages for p in t.pools] == [24, 9]

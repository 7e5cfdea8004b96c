"""The cache's bookkeeping: no slot or page lost, held twice or freed twice; windows
release what no query can reach; groups have storage of their own."""
import numpy as np
import pytest

from ithaca_b200.cache import (CacheError, CacheFull, KVGroupLayout, KVRequest, PagePool, SequenceCache, SlotTable,
                               StateRequest, plan_groups)


def test_page_pool_never_hands_a_page_out_twice():
    pool = PagePool(5)
    got = [pool.take() for _ in range(5)]
    assert sorted(got) == [0, 1, 2, 3, 4]
    with pytest.raises(CacheFull):
        pool.take()
    pool.give_back(got[2])
    with pytest.raises(CacheError, match="freed twice"):
        pool.give_back(got[2])
    with pytest.raises(CacheError):
        pool.give_back(7)
    assert pool.take() == got[2] and pool.n_free == 0 and pool.held() == 5


def table(n_pages=8, slots=4, window=None):
    return SlotTable([KVGroupLayout(2, 16, window, (0, 1))], [n_pages], slots, 64)


def test_slots_are_given_back_and_used_again():
    t = table()
    a, b = t.alloc_slot(), t.alloc_slot()
    t.reserve(a, 100); t.commit(a, 100)
    t.reserve(b, 64); t.commit(b, 64)
    assert t.pools[0].n_free == 8 - 2 - 1 and t.length[a] == 100
    t.check_consistent()
    t.free_slot(a)
    with pytest.raises(CacheError, match="not in use"):
        t.free_slot(a)
    with pytest.raises(CacheError):
        t.reserve(a, 1)
    c = t.alloc_slot()
    assert c == a and t.length[c] == 0 and t.pools[0].n_free == 7
    assert (t.tables[0][c] == -1).all()
    t.check_consistent()
    for _ in range(2):
        t.alloc_slot()
    with pytest.raises(CacheFull):
        t.alloc_slot()


def test_growth_takes_a_page_only_at_a_boundary_and_full_means_full():
    t = table(n_pages=3, slots=2)
    s = t.alloc_slot()
    t.reserve(s, 64); t.commit(s, 64)
    assert t.pools[0].n_free == 2
    t.reserve(s, 1); t.commit(s, 1)
    assert t.pools[0].n_free == 1
    for _ in range(63):
        t.reserve(s, 1); t.commit(s, 1)
    assert t.pools[0].n_free == 1 and t.length[s] == 128
    u = t.alloc_slot()
    t.reserve(u, 10)
    before = t.tables[0].copy()
    with pytest.raises(CacheFull):
        t.reserve(s, 1)
    assert (t.tables[0] == before).all()
    with pytest.raises(CacheError, match="reserved"):
        t.commit(u, 65)
    t.check_consistent()


def test_random_traffic_keeps_the_books():
    rng = np.random.default_rng(0)
    t = SlotTable([KVGroupLayout(2, 16, None, (0,)), KVGroupLayout(1, 32, 100, (1,))], [40, 40], 6, 64)
    live = {}
    for step in range(2000):
        r = rng.random()
        if r < 0.15 and len(live) < 6:
            live[t.alloc_slot()] = 0
        elif r < 0.25 and live:
            s = list(live)[rng.integers(len(live))]
            t.free_slot(s); del live[s]
        elif live:
            s = list(live)[rng.integers(len(live))]
            n = int(rng.integers(1, 90))
            try:
                t.reserve(s, n)
            except CacheFull:
                continue
            t.commit(s, n); live[s] += n
            assert t.length[s] == live[s]
        if step % 50 == 0:
            t.check_consistent()
    for s in list(live):
        t.free_slot(s)
    t.check_consistent()
    assert all(p.n_free == p.n_pages for p in t.pools) and t.n_slots_in_use() == 0


def test_a_window_releases_pages_no_query_can_reach():
    t = table(n_pages=6, slots=1, window=100)
    s = t.alloc_slot()
    t.reserve(s, 300); t.commit(s, 300)           # the next query (position 300) reaches back to 201
    row = t.tables[0][s]
    assert list(row[:3] == -1) == [True, True, True] and row[3] >= 0 and row[4] >= 0
    assert t.pools[0].n_free == 4
    for _ in range(60):
        t.reserve(s, 1); t.commit(s, 1)           # length 360: reaches back to 261 -> page 3 (192..255) is dead
    assert t.tables[0][s][3] == -1 and t.pools[0].n_free == 4
    with pytest.raises(CacheError, match="released"):
        t.truncate(s, 200)
    assert t.length[s] == 360                      # a refusal changes nothing
    with pytest.raises(CacheError, match="released"):
        t.truncate(s, 330)                         # position 330 reaches back to 231, which lay in page 3
    t.truncate(s, 356)                             # position 356 reaches back to 257: page 4 is still there
    assert t.length[s] == 356
    t.reserve(s, 30); t.commit(s, 30)
    t.check_consistent()
    t.truncate(s, 0)                               # back to the start: every page goes back, the slot stays
    assert t.length[s] == 0 and t.pools[0].n_free == 6 and t.in_use(s)
    t.reserve(s, 130); t.commit(s, 130)
    assert list(t.tables[0][s][:3] >= 0) == [True, True, True]
    t.check_consistent()
    t.free_slot(s)
    assert t.pools[0].n_free == 6


def test_truncate_keeps_a_prefix():
    t = table()
    s = t.alloc_slot()
    t.reserve(s, 200); t.commit(s, 200)
    t.truncate(s, 70)
    assert t.length[s] == 70 and t.pools[0].n_free == 8 - 4
    t.reserve(s, 100); t.commit(s, 100)
    assert t.pools[0].n_free == 8 - 4 and t.length[s] == 170
    with pytest.raises(CacheError):
        t.truncate(s, 171)


def test_groups_by_need_and_fixed_size_state():
    req = {0: [KVRequest(2, 16, None)], 1: [KVRequest(2, 16, 50)], 2: [KVRequest(2, 16, None)],
           3: [StateRequest("h", (4, 8))], 4: [KVRequest(1, 32, None), StateRequest("h", (4, 8))]}
    kv, st = plan_groups(req)
    assert [(g.n_kv_heads, g.head_dim, g.window, g.cache_entries) for g in kv] == \
        [(2, 16, None, (0, 2)), (2, 16, 50, (1,)), (1, 32, None, (4,))]
    assert [(s.name, s.shape, s.cache_entries) for s in st] == [("h", (4, 8), (3, 4))]
    c = SequenceCache(req, max_tokens=640, device=None)
    assert c.n_pages == 10 and c.max_slots == 10 and len(c.table.pools) == 3
    assert c.layer(1).kv_group == 1 and c.layer(1).window == 50 and c.layer(3).kv_group is None
    s = c.alloc_slot()
    c.reserve([s], [130]); c.commit([s], [130])
    assert [p.n_free for p in c.table.pools] == [7, 8, 7]          # the windowed group already released a page
    with pytest.raises(CacheError, match="fixed-size state"):
        c.truncate(s, 5)
    c.free_slot(s)
    with pytest.raises(CacheError):
        plan_groups({0: [KVRequest(1, 16), KVRequest(1, 16)]})


def test_a_step_reserves_for_all_or_for_none():
    c = SequenceCache({0: [KVRequest(1, 16)]}, max_tokens=256, device=None)
    a, b = c.alloc_slot(), c.alloc_slot()
    with pytest.raises(CacheFull):
        c.reserve([a, b], [129, 129])
    assert c.table.pools[0].n_free == 4
    c.reserve([a, b], [128, 128])
    assert c.table.pools[0].n_free == 0

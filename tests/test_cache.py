"""Slots and pages: nothing lost, nothing held twice, nothing freed twice (no GPU)."""
import random

import numpy as np
import pytest

from herbert_rs_b200.cache import CacheNeed, IdPool, KVNeed, SequenceCache, StateNeed
from herbert_rs_b200.errors import CacheError


def test_pool_gives_lowest_free_id_and_refuses_double_free():
    p = IdPool(4, "slot")
    assert [p.alloc() for _ in range(4)] == [0, 1, 2, 3]
    with pytest.raises(CacheError, match="no free slot"):
        p.alloc()
    p.free(2); p.free(0)
    with pytest.raises(CacheError, match="freed twice"):
        p.free(2)
    with pytest.raises(CacheError, match="does not exist"):
        p.free(7)
    assert p.alloc() == 0 and p.alloc() == 2
    p.check()


def _cache(pages=8, slots=4, window=None, state=False, page=16, max_seq_len=None):
    needs = [CacheNeed(kv=KVNeed(2, 16)), CacheNeed(kv=KVNeed(2, 16, window)),
             CacheNeed(kv=KVNeed(2, 16), state=StateNeed((3,)) if state else None)]
    return SequenceCache(needs, [None, None, None], pages, slots, page_size=page, max_seq_len=max_seq_len)


def test_groups_by_need():
    c = _cache(window=20)
    assert c.num_kv_groups == 2
    assert c.step_kv == [(0, 0, True), (1, 0, True), (0, 1, True)]
    c2 = _cache()
    assert c2.num_kv_groups == 1 and [e for _, e, _ in c2.step_kv] == [0, 1, 2]


def test_step_reading_another_steps_cache():
    needs = [CacheNeed(kv=KVNeed(2, 16)), CacheNeed(kv=KVNeed(2, 16))]
    c = SequenceCache(needs, [None, 0], 4, 2, page_size=16)
    assert c.step_kv == [(0, 0, True), (0, 0, False)]
    assert len(c._kv_entries[0]) == 1          # the reader has no storage of its own
    with pytest.raises(CacheError, match="earlier step"):
        SequenceCache(needs, [1, None], 4, 2, page_size=16)


def test_reserve_advance_free_cycle():
    c = _cache(pages=8, slots=3)
    a, b = c.alloc_slot(), c.alloc_slot()
    c.reserve([(a, 17), (b, 1)])
    assert len(c.pages_of(a, 0)) == 2 and len(c.pages_of(b, 0)) == 1
    c.advance(a, 17); c.advance(b, 1)
    c.reserve([(a, 1), (b, 15)])           # b fills its page exactly, a stays inside its second
    assert c.pools[0].held_count == 3
    c.advance(a, 1); c.advance(b, 15)
    c.reserve([(b, 1)])
    assert len(c.pages_of(b, 0)) == 2
    c.check()
    rows = c.page_rows(0, [b, a], 4)
    assert rows.dtype == np.int32 and rows.shape == (2, 4)
    assert list(rows[1][:2]) == c.pages_of(a, 0)
    c.free_slot(a)
    with pytest.raises(CacheError, match="not held"):
        c.free_slot(a)
    with pytest.raises(CacheError, match="not held"):
        c.reserve([(a, 1)])
    c.free_slot(b)
    assert c.pools[0].free_count == 8 and c.slots.free_count == 3
    c.check()


def test_refusals_leave_the_cache_unchanged():
    c = _cache(pages=4, slots=2, max_seq_len=40)
    a, b = c.alloc_slot(), c.alloc_slot()
    with pytest.raises(CacheError, match="twice in one step"):
        c.reserve([(a, 1), (a, 1)])
    with pytest.raises(CacheError, match="exceed the limit of 40"):
        c.reserve([(a, 41)])
    with pytest.raises(CacheError, match="at least one token"):
        c.reserve([(a, 0)])
    with pytest.raises(CacheError, match="cache full"):
        c.reserve([(a, 40), (b, 40)])      # 3 + 3 pages > 4
    assert c.pools[0].free_count == 4 and c.pages_of(a, 0) == []
    with pytest.raises(CacheError, match="no free slot"):
        c.alloc_slot()
    c.check()


def test_freed_pages_and_slots_are_used_again():
    c = _cache(pages=6, slots=2)
    for round_ in range(5):
        s1, s2 = c.alloc_slot(), c.alloc_slot()
        assert {s1, s2} == {0, 1}
        c.reserve([(s1, 33), (s2, 40)])
        c.advance(s1, 33); c.advance(s2, 40)
        assert c.length(s1) == 33
        c.free_slot(s1)                      # the shorter one ends earlier
        s3 = c.alloc_slot()
        assert s3 == s1 and c.length(s3) == 0 and c.pages_of(s3, 0) == []
        c.reserve([(s3, 48)]); c.advance(s3, 48)
        c.check()
        c.free_slot(s2); c.free_slot(s3)
    assert c.pools[0].free_count == 6


def test_window_group_gives_pages_back_early():
    c = _cache(pages=10, slots=1, window=20)
    s = c.alloc_slot()
    c.reserve([(s, 70)]); c.advance(s, 70)
    # next query at 70 reads keys 51..70 -> logical pages 0..2 (positions < 48) are out of reach
    assert c.pages_of(s, 1)[:3] == [-1, -1, -1] and c.pages_of(s, 1)[3] >= 0
    assert all(p >= 0 for p in c.pages_of(s, 0))
    assert c.pools[1].held_count == 2 and c.pools[0].held_count == 5
    with pytest.raises(CacheError, match="already given back"):
        c.truncate(s, 50)
    c.check()
    c.free_slot(s)
    assert c.pools[1].free_count == 10
    c.check()


def test_truncate():
    c = _cache(pages=8, slots=1)
    s = c.alloc_slot()
    c.reserve([(s, 50)]); c.advance(s, 50)
    c.truncate(s, 18)
    assert c.length(s) == 18 and len(c.pages_of(s, 0)) == 2 and c.pools[0].held_count == 2
    with pytest.raises(CacheError, match="cannot truncate"):
        c.truncate(s, 19)
    c.check()
    c2 = _cache(state=True)
    s2 = c2.alloc_slot()
    c2.reserve([(s2, 5)]); c2.advance(s2, 5)
    with pytest.raises(CacheError, match="cannot be rolled back"):
        c2.truncate(s2, 3)


def test_state_region_exists_even_when_empty():
    c = _cache()
    assert c.state_needs == [] and c.view(0).state is None and c.step_state == [None, None, None]
    c2 = _cache(state=True)
    assert c2.state_needs == [StateNeed((3,))] and c2.step_state[2] == (0, 0)


def test_random_traffic_keeps_invariants():
    rng = random.Random(0)
    c = _cache(pages=40, slots=6, window=24)
    live = {}
    for _ in range(600):
        r = rng.random()
        if r < 0.3 and c.slots.free_count:
            live[c.alloc_slot()] = 0
        elif r < 0.8 and live:
            s = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 5, 17, 40])
            try:
                c.reserve([(s, n)])
                c.advance(s, n)
                live[s] += n
            except CacheError:
                pass
        elif live:
            s = rng.choice(list(live))
            c.free_slot(s)
            del live[s]
        c.check()
        for s, n in live.items():
            assert c.length(s) == n
    for s in list(live):
        c.free_slot(s)
    assert all(p.free_count == 40 for p in c.pools) and c.slots.free_count == 6

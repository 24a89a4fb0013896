"""The cache's book-keeping on the host: no slot or page lost, held twice or freed twice; groups;
rings; reservations all-or-nothing (no GPU; storage is not allocated)."""
import random

import pytest

from rust_deeplearning_b200.cache.cache import (Cache, CacheError, KVRequirement, PagePool, RunNeeds, StateRequirement,
                                                ring_pages_for)

GLOBAL = KVRequirement(2, 16, None)
LOCAL = KVRequirement(2, 16, 8)


def make(max_tokens=64, max_seqs=4, page_size=4, needs=None, **kw):
    needs = needs or [RunNeeds(LOCAL), RunNeeds(GLOBAL), RunNeeds(LOCAL), RunNeeds(GLOBAL)]
    return Cache(needs, max_tokens=max_tokens, max_seqs=max_seqs, page_size=page_size, allocate=False, **kw)


def invariant(c: Cache):
    """Every page is either free or in exactly one slot's list; every slot is free or live."""
    for g in c.kv_groups:
        held = [p for pages in g.pages.values() for p in pages]
        assert len(held) == len(set(held)), "a page is held twice"
        assert len(held) + g.pool.n_free == g.pool.n_pages, "a page is lost"
        assert set(g.pages) <= set(c.live_slots())
    assert len(c.live_slots()) + c.n_free_slots == c.max_seqs


def test_page_pool():
    p = PagePool(5)
    a = p.take(3)
    assert len(set(a)) == 3 and p.n_free == 2
    with pytest.raises(CacheError):
        p.take(3)
    p.give_back(a[:1])
    with pytest.raises(CacheError):
        p.give_back(a[:1])                       # freed twice
    with pytest.raises(CacheError):
        p.give_back([99])
    assert p.n_free == 3


def test_groups_are_formed_by_need():
    c = make()
    assert len(c.kv_groups) == 2
    by_window = {g.requirement.window: g for g in c.kv_groups}
    assert by_window[None].runs == [1, 3] and by_window[8].runs == [0, 2]
    assert by_window[8].is_ring and by_window[8].ring_pages == ring_pages_for(8, 4) == 3
    assert not by_window[None].is_ring and by_window[None].table_width == 16
    assert c.run_cache(0).kv_group != c.run_cache(1).kv_group and c.run_cache(0).ring_pages == 3
    # a window as long as the context needs no ring
    assert not make(needs=[RunNeeds(KVRequirement(1, 8, 1000))]).kv_groups[0].is_ring


def test_ring_never_overwrites_a_visible_position():
    for page in (1, 4, 16, 64):
        for window in (1, 2, 7, 8, 63, 64, 65, 4096):
            ring_rows = ring_pages_for(window, page) * page
            for p in range(0, 3 * ring_rows, max(1, ring_rows // 7)):
                # writing position p lands on the row of p - ring_rows: no query at q >= p may see it
                assert p - ring_rows < p - window + 1


def test_slots_and_pages_are_reused_and_nothing_is_lost():
    c = make(max_tokens=96, max_seqs=3)
    rng = random.Random(0)
    live = {}
    for _ in range(400):
        invariant(c)
        op = rng.random()
        if op < 0.3 and c.n_free_slots:
            live[c.alloc_slot()] = 0
        elif op < 0.8 and live:
            s = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 5, 17])
            try:
                c.reserve([s], [n])
            except CacheError:
                continue
            c.advance([s], [n])
            live[s] += n
            assert c.length(s) == live[s]
        elif live:
            s = rng.choice(list(live))
            c.free_slot(s)
            del live[s]
    for s in list(live):
        c.free_slot(s)
    invariant(c)
    assert all(g.pool.n_free == g.pool.n_pages for g in c.kv_groups) and c.n_free_slots == 3


def test_errors_change_nothing():
    c = make(max_tokens=32, max_seqs=2)
    a, b = c.alloc_slot(), c.alloc_slot()
    with pytest.raises(CacheError):
        c.alloc_slot()                                            # no free slot
    c.reserve([a, b], [10, 10]); c.advance([a, b], [10, 10])
    before = [(g.pool.n_free, {s: list(p) for s, p in g.pages.items()}) for g in c.kv_groups]
    with pytest.raises(CacheError):
        c.reserve([a, b], [2, 20])                                # b does not fit: a must not grow either
    with pytest.raises(CacheError):
        c.reserve([a, a], [1, 1])                                 # a slot twice in one step
    with pytest.raises(CacheError):
        c.reserve([a], [0])
    assert before == [(g.pool.n_free, {s: list(p) for s, p in g.pages.items()}) for g in c.kv_groups]
    c.free_slot(a)
    with pytest.raises(CacheError):
        c.free_slot(a)                                            # freed twice
    with pytest.raises(CacheError):
        c.length(a)
    with pytest.raises(CacheError):
        c.reserve([a], [1])
    invariant(c)


def test_a_window_group_holds_at_most_its_ring():
    c = make(max_tokens=256, max_seqs=2, max_context=200)
    s = c.alloc_slot()
    c.reserve([s], [150]); c.advance([s], [150])
    local = next(g for g in c.kv_groups if g.is_ring)
    glob = next(g for g in c.kv_groups if not g.is_ring)
    assert len(local.pages[s]) == 3 and len(glob.pages[s]) == 38
    assert c.tokens_held() == 152
    with pytest.raises(CacheError):
        c.reserve([s], [51])                                      # beyond the longest context
    rows = glob.table_rows([s, s], n_rows=4)
    assert rows.shape == (4, glob.table_width) and list(rows[0, :38]) == glob.pages[s] and not rows[2:].any()


def test_reading_another_runs_cache_and_fixed_state():
    needs = [RunNeeds(GLOBAL), RunNeeds(GLOBAL, reads_cache_of=0), RunNeeds(None, StateRequirement((3, 5))),
             RunNeeds(GLOBAL, StateRequirement((3, 5)))]
    c = make(needs=needs)
    assert c.kv_groups[0].runs == [0, 3]                          # the reading run has no storage of its own
    assert c.run_cache(1).kv_group == c.run_cache(0).kv_group and not c.run_cache(1).owns_kv and c.run_cache(0).owns_kv
    assert c.run_cache(2).kv_group is None
    assert c.state_groups[0].runs == [2, 3]
    with pytest.raises(CacheError):
        make(needs=[RunNeeds(GLOBAL, reads_cache_of=0)])
    with pytest.raises(CacheError):
        make(needs=[RunNeeds(None), RunNeeds(GLOBAL, reads_cache_of=0)])


def test_state_is_zeroed_when_a_slot_is_handed_out():
    import torch
    c = Cache([RunNeeds(None, StateRequirement((2,)))], max_tokens=8, max_seqs=2, page_size=4, device="cpu",
              dtype=torch.float32)
    s = c.alloc_slot()
    c.run_cache(0).state[s] += 7
    c.free_slot(s)
    s2 = c.alloc_slot()
    assert s2 == s and not c.run_cache(0).state[s2].any()

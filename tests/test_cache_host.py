"""The cache's bookkeeping: no page or slot lost, held twice or freed twice (no GPU)."""
import random

import pytest

from mynah_slm_b200.cache.pages import PAGE_TOKENS, CacheError, GroupPlan, PagePool, SequencePages, SlotTable


def test_pool_take_and_give_back():
    p = PagePool(4)
    a = p.take(3, owner=0)
    assert len(set(a)) == 3 and p.n_free == 1
    with pytest.raises(CacheError, match="full"):
        p.take(2, owner=1)
    p.give_back(a[:1], owner=0)
    with pytest.raises(CacheError, match="is free"):
        p.give_back(a[:1], owner=0)                 # freed twice
    with pytest.raises(CacheError, match="belongs to slot 0"):
        p.give_back(a[1:2], owner=1)                # not the owner
    assert p.take(1, owner=2) == a[:1]              # the page just freed is the next handed out


def test_slots():
    s = SlotTable(2)
    a, b = s.take(), s.take()
    assert a != b
    with pytest.raises(CacheError, match="in use"):
        s.take()
    s.give_back(a)
    with pytest.raises(CacheError, match="not in use"):
        s.give_back(a)
    assert s.take() == a


def _check_invariants(sp: SequencePages):
    for g, pool in enumerate(sp.pools):
        held = []
        for slot in sp.live_slots():
            pages, base = sp.held(slot, g)
            held += pages
            for pg in pages:
                assert pool.owner(pg) == slot
            # every position a later query can see has a page
            n, w = sp.length[slot], sp.groups[g].window
            first_visible = 0 if w is None else max(0, n - w + 1)
            assert base * PAGE_TOKENS <= first_visible or n == 0 or len(pages) == 0 and n == 0
            assert (base + len(pages)) * PAGE_TOKENS >= n
        assert len(held) == len(set(held)), "a page is held twice"
        assert len(held) + pool.n_free == pool.n_pages, "a page is lost"
    assert len(sp.live_slots()) + sp.slots.n_free == sp.slots.n_slots


def test_random_traffic_keeps_the_books():
    rng = random.Random(0)
    sp = SequencePages([GroupPlan(2, 16, None), GroupPlan(2, 16, 100)], n_pages=40, max_seqs=6)
    live = []
    for _ in range(3000):
        op = rng.random()
        if op < 0.2 and sp.slots.n_free:
            live.append(sp.open())
        elif op < 0.3 and live:
            sp.close(live.pop(rng.randrange(len(live))))
        elif live:
            s = rng.choice(live)
            n = rng.choice([1, 1, 1, 5, 64, 130])
            try:
                sp.reserve(s, n)
            except CacheError:
                sp.close(s); live.remove(s)
                continue
            sp.commit(s, n)
        _check_invariants(sp)
    for s in live:
        sp.close(s)
    _check_invariants(sp)
    assert all(p.n_free == p.n_pages for p in sp.pools)


def test_page_count_is_tokens_rounded_up_to_64():
    sp = SequencePages([GroupPlan(1, 16, None)], n_pages=3, max_seqs=4)
    a = sp.open()
    sp.reserve(a, 64); sp.commit(a, 64)
    assert len(sp.held(a, 0)[0]) == 1
    sp.reserve(a, 1); sp.commit(a, 1)                 # 65 tokens: two pages
    assert len(sp.held(a, 0)[0]) == 2
    b = sp.open()
    sp.reserve(b, 64); sp.commit(b, 64)
    with pytest.raises(CacheError, match="full"):
        sp.reserve(b, 1)                              # 3 pages hold 128 + 64, not one more
    assert len(sp.held(b, 0)[0]) == 1                 # a refused reservation takes nothing
    sp.close(a)
    sp.reserve(b, 1)


def test_window_group_gives_pages_back_early():
    sp = SequencePages([GroupPlan(1, 16, None), GroupPlan(1, 16, 40)], n_pages=8, max_seqs=2)
    s = sp.open()
    sp.reserve(s, 200); sp.commit(s, 200)
    full, base_full = sp.held(s, 0)
    win, base_win = sp.held(s, 1)
    assert len(full) == 4 and base_full == 0
    # next query is position 200 and sees 161..200: pages 2 (128..191) and 3
    assert base_win == 2 and len(win) == 2
    for _ in range(60):
        sp.reserve(s, 1); sp.commit(s, 1)
    assert sp.held(s, 1)[1] == (260 - 40 + 1) // 64
    sp.close(s)
    assert all(p.n_free == 8 for p in sp.pools)


def test_commit_without_pages_is_refused():
    sp = SequencePages([GroupPlan(1, 16, None)], n_pages=2, max_seqs=1)
    s = sp.open()
    with pytest.raises(CacheError, match="without pages"):
        sp.commit(s, 1)
    with pytest.raises(CacheError, match="not open"):
        sp.close(5)

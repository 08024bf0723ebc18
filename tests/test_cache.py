"""The cache's bookkeeping: slots and pages are never lost, held twice or freed twice (no GPU)."""
import random

import numpy as np
import pytest

from rocmforge_b200.cache import CacheError, FreeList, KVRequest, SequenceCache, StateRequest, pages_for


def make(max_tokens=64 * 10, windows=(None, None, 24), max_slots=None, max_seq_len=None, state=False):
    req = {i: KVRequest(2, 16, w) for i, w in enumerate(windows)}
    if state:
        req[len(windows)] = StateRequest.of(acc=(4,), count=((1,), None))
    return SequenceCache(req, max_tokens=max_tokens, max_slots=max_slots, max_seq_len=max_seq_len)


def invariant(c: SequenceCache):
    """Every page is either free or held by exactly one live slot of its group."""
    for g in c.groups:
        held = []
        for s in range(c.max_slots):
            pages = g.held_pages(s)
            if not c.slots.is_held(s):
                assert pages == [], f"freed slot {s} still holds pages {pages}"
            held += pages
        assert len(held) == len(set(held)), "a page is held twice"
        assert len(held) + g.pool.n_free == g.n_pages, "a page was lost"
        for p in held:
            assert g.pool.is_held(p)
        # the device table mirrors the host table wherever a page is held
        t = g.table_dev.numpy()
        mask = g.table >= 0
        assert (t[mask] == g.table[mask]).all()


def test_free_list():
    f = FreeList(3, "thing")
    a, b, c = f.take(), f.take(), f.take()
    assert (a, b, c) == (0, 1, 2) and f.n_free == 0
    with pytest.raises(CacheError):
        f.take()
    f.give_back(1)
    with pytest.raises(CacheError):
        f.give_back(1)                     # freed twice
    with pytest.raises(CacheError):
        f.give_back(7)                     # does not exist
    assert f.take() == 1                   # reused at once


def test_groups_by_need():
    c = make(windows=(None, 24, None, 24, 8))
    keys = sorted((g.window or 0, tuple(g.owners)) for g in c.groups)
    assert keys == [(0, (0, 2)), (8, (4,)), (24, (1, 3))]
    v = c.kv_view(3)
    assert v.window == 24 and tuple(v.k_pages.shape) == (c.n_pages, 2, 64, 16)
    assert c.kv_view(1).k_pages.data_ptr() != v.k_pages.data_ptr()
    assert c.kv_view(1).block_table.data_ptr() == v.block_table.data_ptr()


def test_lengths_pages_and_reuse():
    c = make()
    a, b = c.alloc_slot(), c.alloc_slot()
    starts = c.prepare([a, b], [70, 5])
    assert starts.tolist() == [0, 0]
    c.commit([a, b], [70, 5])
    assert (c.length(a), c.length(b)) == (70, 5)
    full = next(g for g in c.groups if g.window is None)
    assert len(full.held_pages(a)) == 2 and len(full.held_pages(b)) == 1
    invariant(c)
    c.prepare([b], [1]); c.commit([b], [1])
    assert c.length(b) == 6 and len(full.held_pages(b)) == 1
    pages_a = set(full.held_pages(a))
    c.free_slot(a)
    invariant(c)
    with pytest.raises(CacheError):
        c.free_slot(a)                     # freed twice
    with pytest.raises(CacheError):
        c.prepare([a], [1])                # not held
    a2 = c.alloc_slot()
    assert a2 == a and c.length(a2) == 0   # the slot comes back, empty
    c.prepare([a2], [130]); c.commit([a2], [130])
    assert pages_a & set(full.held_pages(a2)), "freed pages are used again"
    invariant(c)


def test_window_group_drops_old_pages():
    c = make(max_tokens=64 * 8, windows=(None, 24))
    s = c.alloc_slot()
    win = next(g for g in c.groups if g.window == 24)
    full = next(g for g in c.groups if g.window is None)
    c.prepare([s], [200]); c.commit([s], [200])
    # the next query (position 200) sees keys >= 177: pages 0 and 1 are gone, 2 and 3 stay
    assert [int(x) >= 0 for x in win.table[s, :4]] == [False, False, True, True]
    assert len(full.held_pages(s)) == 4
    for _ in range(120):
        c.prepare([s], [1]); c.commit([s], [1])
    assert c.length(s) == 320
    assert [int(x) >= 0 for x in win.table[s, :5]] == [False, False, False, False, True]
    assert len(win.held_pages(s)) == 1 and len(full.held_pages(s)) == 5
    invariant(c)
    c.free_slot(s)
    assert win.pool.n_free == win.n_pages and full.pool.n_free == full.n_pages


def test_exhaustion_takes_nothing():
    c = make(max_tokens=64 * 3, windows=(None,))
    a, b = c.alloc_slot(), c.alloc_slot()
    c.prepare([a], [64]); c.commit([a], [64])
    before = c.free_pages()
    with pytest.raises(CacheError) as e:
        c.prepare([a, b], [64, 65])        # needs 1 + 2 pages, 2 are free
    assert "pages" in str(e.value)
    assert c.free_pages() == before and c.length(b) == 0
    invariant(c)
    c.prepare([a, b], [64, 64])            # fits exactly
    c.commit([a, b], [64, 64])
    assert c.free_pages() == [0]
    with pytest.raises(CacheError):
        c.alloc_slot() and c.prepare([2], [1])


def test_step_rules():
    c = make(max_seq_len=100)
    s = c.alloc_slot()
    with pytest.raises(CacheError):
        c.prepare([s, s], [1, 1])          # a slot twice in one step
    with pytest.raises(CacheError):
        c.prepare([s], [0])
    with pytest.raises(CacheError):
        c.prepare([s], [101])              # longer than a sequence may get
    c.prepare([s], [100]); c.commit([s], [100])
    with pytest.raises(CacheError):
        c.prepare([s], [1])
    assert c.max_seq_len == 100


def test_slots_run_out_and_come_back():
    c = make(max_slots=2)
    a, b = c.alloc_slot(), c.alloc_slot()
    with pytest.raises(CacheError):
        c.alloc_slot()
    c.free_slot(a)
    assert c.alloc_slot() == a and c.live_slots == 2
    c.free_slot(a); c.free_slot(b)
    assert c.live_slots == 0


def test_state_is_zero_on_a_fresh_slot():
    c = make(state=True)
    s = c.alloc_slot()
    st = c.state_view(3)
    assert tuple(st["acc"].shape) == (c.max_slots, 4)
    st["acc"][s] += 5.0
    st["count"][s] += 2
    c.free_slot(s)
    s2 = c.alloc_slot()
    assert s2 == s and float(st["acc"][s2].abs().sum()) == 0 and float(st["count"][s2].sum()) == 0
    assert c.view(3) is st and c.view(0).window is None and c.view(99) is None


def test_random_walk_keeps_the_books():
    rng = random.Random(3)
    c = make(max_tokens=64 * 40, windows=(None, 24, 100), max_slots=9)
    live = {}
    for _ in range(600):
        r = rng.random()
        if r < 0.25 and c.slots.n_free:
            s = c.alloc_slot()
            assert s not in live
            live[s] = 0
        elif r < 0.4 and live:
            s = rng.choice(list(live))
            c.free_slot(s)
            del live[s]
        elif live:
            pick = rng.sample(list(live), rng.randint(1, len(live)))
            n = [rng.choice([1, 1, 1, 7, 64, 90]) for _ in pick]
            try:
                c.prepare(pick, n)
            except CacheError:
                invariant(c)
                continue
            c.commit(pick, n)
            for s, k in zip(pick, n):
                live[s] += k
        for s, n_tok in live.items():
            assert c.length(s) == n_tok
            for g in c.groups:
                lo = 0 if g.window is None else max(n_tok - g.window + 1, 0) // 64
                want = set(range(lo, pages_for(n_tok)))
                have = set(np.nonzero(g.table[s] >= 0)[0].tolist())
                assert want <= have, "a page a future query needs is missing"
                if g.window is not None:
                    assert have == want
        invariant(c)
    for s in list(live):
        c.free_slot(s)
    assert all(g.pool.n_free == g.n_pages for g in c.groups) and c.live_slots == 0


def test_epoch_grows_with_every_slot_handed_out_or_given_back():
    c = make()
    e0 = c.epoch
    s = c.alloc_slot()
    assert c.epoch > e0
    e1 = c.epoch
    c.prepare([s], [10]); c.commit([s], [10])
    assert c.epoch == e1, "steps do not change the set of sequences"
    c.free_slot(s)
    assert c.epoch > e1


def test_device_table_names_no_free_page_after_free_and_refill():
    """A sequence ends exactly on a page border after the page for its next position was taken; the slot is
    freed and filled again with a prompt of the same length while another slot stays alive (so the free list
    hands out other pages): wherever the device table still names a page, it is the host table's page, and
    entries of pages given back are cleared with the next upload."""
    c = make(max_tokens=64 * 12, windows=(None, 24))
    keep = c.alloc_slot()
    c.prepare([keep], [70]); c.commit([keep], [70])
    s = c.alloc_slot()
    c.prepare([s], [64]); c.commit([s], [64])
    c.prepare([s], [1])                       # a runner takes the page for position 64 ahead of time
    ahead = [g.table[s, 1] for g in c.groups]
    assert all(p >= 0 for p in ahead)
    c.free_slot(s)
    other = c.alloc_slot()                    # takes the lowest pages, among them the ones just freed
    c.prepare([other], [130]); c.commit([other], [130])
    s2 = c.alloc_slot()
    c.prepare([s2], [64]); c.commit([s2], [64])
    for g in c.groups:
        dev = g.table_dev.numpy()
        for slot in range(c.max_slots):
            for p in range(g.max_pages_per_seq):
                if g.table[slot, p] >= 0:
                    assert dev[slot, p] == g.table[slot, p]
                elif dev[slot, p] > 0:
                    # a page the host no longer lists for this slot must not stay named on the device
                    raise AssertionError(f"device table of slot {slot} still names page {dev[slot, p]} at {p}")
    invariant(c)


def test_reserve_takes_nothing_when_not_everything_fits():
    c = make(max_tokens=64 * 6, windows=(None,), max_slots=3)
    a, b = c.alloc_slot(), c.alloc_slot()
    c.prepare([a, b], [10, 10]); c.commit([a, b], [10, 10])
    free = c.free_pages()
    with pytest.raises(CacheError):
        c.reserve([a, b], [64 * 3, 64 * 4])          # 2 + 3 more pages, 4 are free
    assert c.free_pages() == free and [g.held_pages(a) for g in c.groups] == [[0]]
    with pytest.raises(CacheError):
        c.reserve([a], [64 * 7])                     # beyond the longest sequence the cache holds
    assert c.free_pages() == free
    c.reserve([a, b], [64 * 3, 64 * 3])
    assert c.free_pages() == [0]
    invariant(c)


def test_rollback_gives_back_what_a_failed_step_took():
    c = make(max_tokens=64 * 8, windows=(None, 24))
    s = c.alloc_slot()
    c.prepare([s], [70]); c.commit([s], [70])
    free = c.free_pages()
    c.prepare([s], [200])
    assert c.free_pages() != free
    c.rollback([s])
    assert c.free_pages() == free and c.length(s) == 70
    c.prepare([s], [1]); c.commit([s], [1])           # the slot goes on as if nothing had happened
    invariant(c)

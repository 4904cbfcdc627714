"""The cache manager on the host: no page lost, held twice or freed twice under random orders of
requests; all-or-nothing planning; windows give pages back; state slots."""
from __future__ import annotations

import random

import numpy as np
import pytest

from mrun_b200.cache import FREED, CacheManager, FixedState, OutOfPages, PagedKV, PagePool


def manager(pages=32, page_size=4, requests=4, window=None, extra=()):
    needs = [PagedKV(2, 8), PagedKV(2, 8)] + list(extra)
    if window:
        needs.append(PagedKV(1, 8, window=window))
    return CacheManager(needs, [None] * len(needs), page_size, pages, requests)


def test_pool_refuses_double_free_and_is_all_or_nothing():
    pool = PagePool(4)
    a = pool.alloc(3)
    with pytest.raises(OutOfPages):
        pool.alloc(2)
    assert pool.free_count == 1
    pool.free(a[:1])
    with pytest.raises(ValueError, match="twice"):
        pool.free(a[:1])
    with pytest.raises(ValueError, match="outside"):
        pool.free([9])
    pool.check()
    # a page given back is handed out next
    assert pool.alloc(1) == a[:1]


def test_append_commit_release():
    m = manager()
    r = m.admit("a")
    plan = m.plan_append([(r, 9)])
    assert len(r.blocks[("paged", None)]) == 3 and r.pending == 9 and r.length == 0
    m.commit(plan)
    assert r.length == 9 and m.free_pages() == 29
    m.commit(m.plan_append([(r, 3)]))           # fills the third page, takes none
    assert m.free_pages() == 29
    m.commit(m.plan_append([(r, 1)]))
    assert m.free_pages() == 28
    m.check_invariants()
    m.release(r)
    assert m.free_pages() == 32 and m.free_slots == 4
    with pytest.raises(ValueError, match="twice"):
        m.release(r)
    with pytest.raises(ValueError, match="released"):
        m.plan_append([(r, 1)])
    m.check_invariants()


def test_trim_gives_back_the_pages_beyond_the_cut():
    """The reference's trim (crates/mrun-engine/src/ledger.rs:400-441): a request cut back to
    its first n tokens keeps the pages that hold them, gives the others back, and appends from
    n on; not during a step, not beyond its length, and not where a window has passed."""
    m = manager()
    r = m.admit("a")
    m.commit(m.plan_append([(r, 5)]))
    assert m.free_pages() == 30
    plan = m.plan_append([(r, 9)])
    with pytest.raises(ValueError, match="uncommitted"):
        m.trim(r, 2)
    m.commit(plan)                                             # 14 tokens, 4 pages
    assert r.length == 14 and m.free_pages() == 28
    with pytest.raises(ValueError, match="cannot be cut to 15"):
        m.trim(r, 15)
    m.trim(r, 14)                                              # no change
    m.trim(r, 9)                                               # 9 tokens need 3 pages
    assert r.length == 9 and m.free_pages() == 29 and len(r.blocks[("paged", None)]) == 3
    m.commit(m.plan_append([(r, 4)]))                          # goes on from 9
    assert r.length == 13 and m.free_pages() == 28
    m.trim(r, 0)
    assert r.length == 0 and m.free_pages() == 32
    m.commit(m.plan_append([(r, 2)]))
    m.check_invariants()
    m.release(r)
    assert m.free_pages() == 32
    # a group with a window of 6 keys: at 14 tokens it has given back the pages before position 9
    w = manager(window=6)
    r = w.admit("a")
    w.commit(w.plan_append([(r, 14)]))
    with pytest.raises(ValueError, match="window of 6 keys"):
        w.trim(r, 9)                                           # would need keys from position 4 on
    assert r.length == 14
    w.trim(r, 13)                                              # needs keys from position 8 on: still held
    assert r.length == 13
    w.check_invariants()
    # per-request state of fixed size is not rewound
    f = manager(extra=[FixedState((3,))])
    r = f.admit("a")
    f.commit(f.plan_append([(r, 6)]))
    with pytest.raises(ValueError, match="fixed size"):
        f.trim(r, 3)


def test_out_of_pages_changes_nothing():
    m = manager(pages=6)
    a, b = m.admit("a"), m.admit("b")
    m.commit(m.plan_append([(a, 8)]))
    before = (list(a.blocks[("paged", None)]), m.free_pages(), m.groups[("paged", None)].table.copy())
    with pytest.raises(OutOfPages):
        m.plan_append([(a, 4), (b, 16)])         # 1 + 4 pages wanted, 4 free
    assert (list(a.blocks[("paged", None)]), m.free_pages()) == before[:2]
    assert (m.groups[("paged", None)].table == before[2]).all()
    assert a.pending == 0 and b.pending == 0
    m.check_invariants()
    plan = m.plan_append([(a, 4), (b, 12)])
    m.rollback(plan)
    assert m.free_pages() == before[1] and a.pending == 0 and b.blocks[("paged", None)] == []
    m.check_invariants()
    with pytest.raises(ValueError, match="already"):
        m.commit(plan)


def test_a_request_cannot_be_in_a_step_twice_or_skip_a_commit():
    m = manager()
    r = m.admit("a")
    with pytest.raises(ValueError, match="twice"):
        m.plan_append([(r, 1), (r, 1)])
    plan = m.plan_append([(r, 2)])
    with pytest.raises(ValueError, match="uncommitted"):
        m.plan_append([(r, 1)])
    with pytest.raises(ValueError, match="uncommitted"):
        m.release(r)
    m.commit(plan)
    with pytest.raises(ValueError, match="already live"):
        m.admit("a")


def test_window_group_gives_back_what_the_window_has_passed():
    m = manager(pages=64, page_size=4, window=10)
    key_w, key_f = ("paged", 10), ("paged", None)
    r = m.admit("a")
    m.commit(m.plan_append([(r, 30)]))
    # the next token (position 30) sees keys 21..30: blocks 0..4 (positions 0..19) are passed
    assert r.blocks[key_w][:5] == [FREED] * 5 and FREED not in r.blocks[key_w][5:]
    assert FREED not in r.blocks[key_f]
    assert m.free_pages(key_w) == 64 - 3 and m.free_pages(key_f) == 64 - 8
    row = m.groups[key_w].table[r.slot]
    assert list(row[:8]) == r.blocks[key_w]
    for _ in range(20):
        m.commit(m.plan_append([(r, 1)]))
        m.check_invariants()
        held = len(r.pages_held(key_w))
        assert held <= -(-10 // 4) + 1
    m.release(r)
    assert m.free_pages(key_w) == 64 and m.free_pages(key_f) == 64
    m.check_invariants()


def test_state_slots_and_shared_caches():
    needs = [PagedKV(2, 8), FixedState((3, 5)), None]
    shares = [None, None, 0]
    m = CacheManager(needs, shares, 4, 8, 2)
    assert m.entries[2].group_key == ("paged", None) and not m.entries[2].writable and m.entries[0].writable
    assert m.entries[1].need == FixedState((3, 5))
    a, b = m.admit("a"), m.admit("b")
    assert {a.slot, b.slot} == {0, 1}
    with pytest.raises(OutOfPages, match="state slots"):
        m.admit("c")
    m.release(a)
    c = m.admit("c")
    assert c.slot == a.slot
    with pytest.raises(ValueError, match="keeps none"):
        CacheManager([None, None], [None, 0], 4, 8, 2)


def test_block_limit_per_request():
    m = CacheManager([PagedKV(1, 8)], [None], 4, 64, 2, max_blocks_per_request=3)
    r = m.admit("a")
    m.commit(m.plan_append([(r, 12)]))
    with pytest.raises(OutOfPages, match="blocks of request"):
        m.plan_append([(r, 1)])
    m.check_invariants()


def test_table_updates_reach_the_device_copy_in_order():
    m = manager(pages=8, page_size=4)
    key = ("paged", None)
    r = m.admit("a")
    plan = m.plan_append([(r, 6)])
    m.rollback(plan)                              # set then cleared: the last value per index wins
    plan = m.plan_append([(r, 6)])
    m.commit(plan)
    index, value = m.drain_table_updates()[key]
    mirror = np.full(m.groups[key].table.size, FREED, dtype=np.int32)
    mirror[index] = value
    assert (mirror.reshape(m.groups[key].table.shape) == m.groups[key].table).all()
    assert m.drain_table_updates() == {}


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("window", [None, 7])
def test_random_orders_of_requests(seed, window):
    """Admit, append, fail, roll back and release in random order; after every operation every
    page is either free or held by exactly one request, and the tables mirror the block lists."""
    rng = random.Random(seed)
    m = manager(pages=24, page_size=4, requests=5, window=window)
    live, next_id = [], 0
    mirror = {key: np.full(g.table.shape, FREED, dtype=np.int32) for key, g in m.groups.items()}
    for step in range(400):
        action = rng.random()
        if action < 0.25 and m.free_slots:
            live.append(m.admit(next_id))
            next_id += 1
        elif action < 0.8 and live:
            batch = rng.sample(live, rng.randint(1, len(live)))
            items = [(r, rng.choice([1, 1, 1, 2, 5, 9, 17])) for r in batch]
            try:
                plan = m.plan_append(items)
            except OutOfPages:
                assert all(r.pending == 0 for r in live)
            else:
                if rng.random() < 0.2:
                    m.rollback(plan)
                else:
                    m.commit(plan)
        elif action < 0.9 and live:
            # cut a request back: pages beyond the cut go back; a window may refuse
            r = rng.choice(live)
            cut = rng.randint(0, r.length)
            try:
                m.trim(r, cut)
                assert r.length == cut
            except ValueError as error:
                assert window and "window" in str(error)
        elif live:
            victim = live.pop(rng.randrange(len(live)))
            m.release(victim)
        m.check_invariants()
        for key, (index, value) in m.drain_table_updates().items():
            mirror[key].reshape(-1)[index] = value
        for key, g in m.groups.items():
            assert (mirror[key] == g.table).all()
    for r in live:
        m.release(r)
    m.check_invariants()
    assert all(g.pool.free_count == 24 for g in m.groups.values()) and m.free_slots == 5

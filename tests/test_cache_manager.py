"""The cache manager: no page lost, held twice or freed twice, under random orders of requests (no GPU)."""
import random

import pytest
import torch

from swifttransformer_b200.cache import CacheManager, PageError, PagePool
from swifttransformer_b200.parts.base import PagedKVSpec, StateSpec


def test_pool_basics():
    p = PagePool(5)
    a = p.alloc(3)
    assert a == [0, 1, 2] and p.num_free == 2
    assert p.alloc(3) is None and p.num_free == 2, "all or nothing"
    p.free([1])
    assert p.alloc(1) == [1], "the page freed last is used again first"
    with pytest.raises(PageError):
        p.free([4])
    p.free([0])
    with pytest.raises(PageError):
        p.free([0])
    p.check()


def manager(specs, page_size=4, num_pages=12, max_seqs=3, max_len=64):
    return CacheManager(specs, torch.float32, "cpu", page_size, num_pages, max_seqs, max_len)


def test_groups_by_need_and_views():
    full, win = PagedKVSpec(2, 8), PagedKVSpec(2, 8, window=6)
    m = manager([full, win, full, StateSpec((3, 2)), None, win])
    assert len(m.groups) == 2
    g_full = next(g for g in m.groups if g.spec.window is None)
    g_win = next(g for g in m.groups if g.spec.window == 6)
    assert g_full.entries == [0, 2] and g_win.entries == [1, 5]
    assert g_full.kv.shape == (12, 2, 2, 2, 4, 8)
    e = m.entries()
    assert e[2].view().layer == 1 and e[2].view().pool is g_full.kv
    assert e[5].view(False).writable is False and e[5].view().layer == 1
    assert e[3].view().state.shape == (3, 3, 2) and e[4].view() is None
    assert m.bytes_per_token() == 2 * (2 * 2 * 2 * 8 * 4)


def test_window_pages_are_given_back_when_passed():
    m = manager([PagedKVSpec(1, 8, window=6)], page_size=4, num_pages=4, max_seqs=2, max_len=64)
    s = m.alloc_slot()
    g = m.groups[0]
    n = 0
    for step in range(40):                    # far more tokens than four pages hold: only the window is kept
        assert m.reserve(s, n, n + 1)
        n += 1
        m.commit(s, n)
        m.check()
        first_needed = max(0, n - 6 + 1) // 4
        assert sorted(g.pages[s]) == list(range(first_needed, (n - 1) // 4 + 1))
    # a long first portion needs all of its pages at once, then drops what the window passed
    s2 = m.alloc_slot()
    assert not m.reserve(s2, 0, 30)
    assert m.free_pages == 4 - len(g.pages[s]), "a failed reservation takes nothing"
    m.free_slot(s)
    assert m.reserve(s2, 0, 16)
    m.commit(s2, 16)
    assert sorted(g.pages[s2]) == [2, 3]
    m.free_slot(s2)
    assert m.free_pages == 4
    m.check()


def test_state_rows_start_at_zero():
    m = manager([StateSpec((4,))], max_seqs=2)
    s = m.alloc_slot()
    st = m.entries()[0].view().state
    st[s] += 5
    m.free_slot(s)
    s2 = m.alloc_slot()
    assert s2 == s and torch.all(st[s2] == 0)
    with pytest.raises(RuntimeError):
        m.free_slot(1 - s2)


def test_block_table_updates_keep_only_the_newest_value_per_entry():
    m = manager([PagedKVSpec(1, 8)], page_size=4, num_pages=3, max_seqs=2)
    s = m.alloc_slot()
    assert m.reserve(s, 0, 8)
    m.free_slot(s)
    s = m.alloc_slot()
    assert m.reserve(s, 0, 4)
    upd = dict(m.groups[0].take_updates())
    row = s * m.max_pages_per_seq
    assert upd[row] == m.groups[0].pages[s][0] and upd[row + 1] == -1
    assert m.groups[0].take_updates() == []


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_nothing(seed):
    rng = random.Random(seed)
    specs = [PagedKVSpec(2, 8), PagedKVSpec(1, 16, window=10), PagedKVSpec(2, 8)]
    m = manager(specs, page_size=4, num_pages=20, max_seqs=4, max_len=80)
    live = {}
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and m.num_free_slots:
            live[m.alloc_slot()] = 0
        elif op < 0.45 and live:
            s = rng.choice(list(live))
            m.free_slot(s)
            del live[s]
        elif live:
            s = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 5, 13])
            if live[s] + n > 80:
                continue
            before = [g.pool.num_free for g in m.groups]
            if m.reserve(s, live[s], live[s] + n):
                live[s] += n
                m.commit(s, live[s])
            else:
                assert [g.pool.num_free for g in m.groups] == before, "a refused reservation takes nothing"
        m.check()
        for g in m.groups:
            for s, n in live.items():
                first = 0 if g.spec.window is None else max(0, n - g.spec.window + 1) // 4
                want = list(range(first, (n - 1) // 4 + 1)) if n else []
                assert sorted(g.pages[s]) == want
    for s in list(live):
        m.free_slot(s)
    m.check()
    assert all(g.pool.num_free == 20 for g in m.groups)

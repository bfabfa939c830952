"""The cache manager on the host: pages, block tables, windows, slots (no GPU)."""
import random

import pytest
import torch

from flint_b200.cache.manager import CacheManager, KVSpec, StateSpec
from flint_b200.cache.pages import NO_PAGE, GroupPages, PagePool
from flint_b200.errors import CacheError


def manager(n_pages=8, page=16, slots=4, ctx=256, window=0, two_groups=False, state=False):
    kv = {0: KVSpec(2, 16, window), 1: KVSpec(2, 16, window)}
    if two_groups:
        kv[2] = KVSpec(2, 16, 32)
    st = {1: StateSpec((3, 5))} if state else {}
    return CacheManager(kv, st, page_size=page, n_pages=n_pages, max_slots=slots, max_context=ctx,
                        dtype=torch.float32, device="cpu")


def test_pool_take_and_give_back():
    p = PagePool(3)
    a, b, c = p.take(), p.take(), p.take()
    assert sorted([a, b, c]) == [0, 1, 2] and p.free_pages == 0
    with pytest.raises(CacheError, match="exhausted"):
        p.take()
    p.give_back(b)
    assert p.take() == b                      # the page just freed is used again
    with pytest.raises(CacheError, match="freed twice"):
        p.give_back(a) or p.give_back(a)
    p.check()


def test_growth_reuse_and_exhaustion():
    m = manager(n_pages=4)
    s0, s1 = m.admit(), m.admit()
    m.ensure(s0, 0, 17)                       # 2 pages
    m.ensure(s1, 0, 16)                       # 1 page
    assert m.free_pages() == 1 and m.pages_needed(s0, 17, 33) == 1 and m.pages_needed(s0, 17, 32) == 0
    m.ensure(s0, 17, 33)
    assert not m.can_run(s1, 16, 17)
    with pytest.raises(CacheError, match="exhausted"):
        m.ensure(s1, 16, 17)
    held = set(m.groups[0].pages.tables[s0].held())
    m.release(s0)
    m.ensure(s1, 16, 40)
    assert set(m.groups[0].pages.tables[s1].held()) & held      # pages of s0 serve s1 now
    m.check()
    with pytest.raises(CacheError, match="released twice"):
        m.release(s0)


def test_context_limit_and_slots():
    m = manager(n_pages=64, ctx=64, slots=2)
    a, b = m.admit(), m.admit()
    with pytest.raises(CacheError, match="no free request slot"):
        m.admit()
    with pytest.raises(CacheError, match="context limit 64"):
        m.ensure(a, 0, 65)
    m.release(b)
    assert m.admit() == b


def test_window_gives_pages_back_and_never_needs_the_far_past():
    m = manager(n_pages=5, page=16, window=40)
    s = m.admit()
    g = m.groups[0].pages
    m.ensure(s, 0, 50)
    assert g.pool.used_pages == 4
    m.advance(s, 50)          # next query at 50 sees keys >= 11: page 0 (0..15) still needed
    assert g.pool.used_pages == 4
    m.ensure(s, 50, 70)
    m.advance(s, 70)          # next query at 70 sees keys >= 31: page 0 is dead
    assert g.tables[s].pages[0] == NO_PAGE and g.pool.used_pages == 4
    # a long run in small steps never holds more than window/page + 2 pages
    pos = 70
    while pos < 250:
        m.ensure(s, pos, pos + 3)
        pos += 3
        m.advance(s, pos)
        assert g.pool.used_pages <= 40 // 16 + 2
    m.check()
    # a request that starts far in (recomputation is always from 0, but the table must cope)
    s2 = m.admit()
    m.release(s)
    m.ensure(s2, 0, 10)
    m.check()


def test_groups_have_pages_of_their_own_and_state_is_zeroed():
    m = manager(n_pages=6, two_groups=True, state=True)
    assert len(m.groups) == 2
    s = m.admit()
    m.state_of(1)[s].fill_(7.0)
    m.ensure(s, 0, 90)
    m.advance(s, 90)
    full, win = (g for g in m.groups if g.spec.window == 0), (g for g in m.groups if g.spec.window)
    full, win = next(full), next(win)
    assert full.pages.pool.used_pages == 6 and win.pages.pool.used_pages == 3
    assert m.view(0).k.shape == (6, 2, 16, 16) and m.view(2).block_table.data_ptr() != m.view(0).block_table.data_ptr()
    assert m.view(0).block_table.data_ptr() == m.view(1).block_table.data_ptr()   # same group, same table
    assert m.view(0).k.data_ptr() != m.view(1).k.data_ptr()                         # own storage per call
    m.release(s)
    s2 = m.admit()
    assert s2 == s and float(m.state_of(1)[s2].abs().sum()) == 0.0                   # zeroed on admission


def test_block_table_reaches_the_device_copy():
    m = manager(n_pages=8)
    s = m.admit()
    m.ensure(s, 0, 40)
    m.sync()
    row = m.view(0).block_table[s].tolist()
    assert row[:3] == m.groups[0].pages.tables[s].pages and all(x == NO_PAGE for x in row[3:])
    m.release(s)
    m.sync()
    assert all(x == NO_PAGE for x in m.view(0).block_table[s].tolist())


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("window", [0, 24])
def test_random_orders_lose_no_page(seed, window):
    """Random admissions, growth, window advances and releases: at every point each page is
    free or held by exactly one request, and at the end all pages are free."""
    rnd = random.Random(seed)
    m = manager(n_pages=12, page=16, slots=4, ctx=200, window=window)
    live = {}
    for _ in range(400):
        op = rnd.random()
        if op < 0.25 and m.free_slots:
            live[m.admit()] = 0
        elif op < 0.85 and live:
            s = rnd.choice(list(live))
            n = rnd.choice([1, 1, 2, 5, 17, 40])
            if live[s] + n <= 200 and m.can_run(s, live[s], live[s] + n):
                m.ensure(s, live[s], live[s] + n)
                live[s] += n
                m.advance(s, live[s])
            else:
                with pytest.raises(CacheError):
                    m.ensure(s, live[s], live[s] + n)
        elif live:
            s = rnd.choice(list(live))
            m.release(s)
            del live[s]
        m.check()
        for g in m.groups:
            for s, n in live.items():
                t = g.pages.tables[s]
                first = g.pages.first_visible(n) // 16 if n else 0
                assert all(p != NO_PAGE for p in t.pages[first:]), "a page a later query needs is missing"
    for s in list(live):
        m.release(s)
    m.check()
    assert all(g.pages.pool.free_pages == 12 for g in m.groups)


def test_truncate():
    g = GroupPages(8, 16, 0, 2, 16)
    g.ensure(0, 0, 70)
    g.truncate(0, 33)
    assert len(g.tables[0].pages) == 3 and g.pool.used_pages == 3
    g.check()

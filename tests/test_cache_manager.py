"""The cache manager's bookkeeping: no page lost, held twice or freed twice, under random orders of
requests; window groups give pages back behind the window; state slots travel with the request."""

import random

import pytest
import torch

from ampere_kv_engine_b200.cache.block_pool import IdPool, OutOfPages
from ampere_kv_engine_b200.cache.manager import CacheManager
from ampere_kv_engine_b200.parts.base import CacheSpec

FULL = CacheSpec("full", 2, 16)
WIN = CacheSpec("window", 2, 16, window=40)


def manager(specs, page=16, pages=16, seqs=4, cache_of=None, storage=False, **kw):
    return CacheManager(specs, cache_of or [None] * len(specs), page_size=page, num_pages=pages, max_seqs=seqs,
                        dtype=torch.float32, device="cpu", allocate_storage=storage, **kw)


def test_pool_is_lifo_and_refuses_double_free():
    pool = IdPool(4)
    assert [pool.allocate() for _ in range(3)] == [0, 1, 2]
    pool.free(1)
    pool.free(0)
    assert pool.allocate() == 0 and pool.allocate() == 1          # returned ids are reused first
    with pytest.raises(ValueError, match="not held"):
        pool.free(3)
    pool.free(2)
    with pytest.raises(ValueError, match="not held"):
        pool.free(2)
    with pytest.raises(ValueError, match="outside"):
        pool.free(9)
    assert pool.allocate_many(2) == [2, 3]
    with pytest.raises(OutOfPages):
        pool.allocate()
    with pytest.raises(OutOfPages):
        IdPool(2).allocate_many(3)


def test_groups_follow_the_mixers_needs():
    m = manager([FULL, WIN, WIN, CacheSpec("none", state_shape=(8,)), FULL], cache_of=[None, None, None, None, 0],
                storage=True)
    assert [(g.spec.kind, g.positions) for g in m.groups] == [("full", [0]), ("window", [1, 2])]
    views = m.layer_views()
    assert views[4].group == 0 and not views[4].writes and views[4].k_cache.data_ptr() == views[0].k_cache.data_ptr()
    assert views[3].group is None and views[3].state.shape == (4, 8)
    assert views[1].k_cache.shape == (16, 2, 16, 16) and views[1].k_cache.data_ptr() != views[2].k_cache.data_ptr()
    with pytest.raises(ValueError, match="another shape"):
        manager([FULL, WIN], cache_of=[None, 0])


def test_reserve_is_all_or_nothing_across_groups():
    m = manager([FULL, WIN], pages=[8, 2])
    s = m.open("a")
    with pytest.raises(OutOfPages):
        m.reserve(s, 40)                       # 3 pages: the window group has only 2
    assert m.free_pages() == [8, 2] and s.pages == [[], []]
    m.reserve(s, 20)
    assert m.free_pages() == [6, 0]
    m.check_invariants()


def test_window_pages_come_back_behind_the_window():
    m = manager([FULL, WIN], pages=32)
    s = m.open("a")
    held = []
    for chunk in (24, 7, 2, 13, 50, 1, 1, 30, 1, 1):
        m.reserve(s, chunk)
        start = s.length
        # every key the step's queries may read is backed by a page
        first_key = max(0, start - 40 + 1)
        for g, lo in ((0, 0), (1, first_key)):
            assert all(s.pages[g][p // 16] >= 0 for p in range(lo, start + chunk))
        m.commit(s, chunk)
        held.append((s.length, len(s.held_pages(0)), len(s.held_pages(1))))
        m.check_invariants()
    assert held[-1][1] == (130 + 15) // 16                       # the full group keeps everything
    assert all(w <= (40 + 15) // 16 + 1 for _, _, w in held)      # the window group only the window
    assert s.pages[1][0] == -1 and s.first_live[1] == (130 - 40 + 1) // 16
    with pytest.raises(ValueError, match="given back"):
        m.slot_of(s, 1, 0)
    assert m.slot_of(s, 1, 129) == s.pages[1][129 // 16] * 16 + 129 % 16
    m.close(s)
    assert m.free_pages() == [32, 32]


def test_close_twice_and_release_unused():
    m = manager([FULL])
    s = m.open("a")
    m.reserve(s, 40)
    m.commit(s, 10)
    m.release_unused(s)
    assert len(s.pages[0]) == 1 and m.free_pages() == [15]
    m.close(s)
    with pytest.raises(ValueError, match="closed before"):
        m.close(s)
    with pytest.raises(ValueError, match="is closed"):
        m.reserve(s, 1)
    t = m.open("a")                                               # the id may be used again
    with pytest.raises(ValueError, match="already holds"):
        m.open("a")
    m.close(t)


def test_state_slots_are_zeroed_and_returned():
    m = manager([CacheSpec("none", state_shape=(3,)), FULL], seqs=2, storage=True)
    a = m.open("a")
    m.state[0][a.state_slot] = 7.0
    b = m.open("b")
    with pytest.raises(OutOfPages):
        m.open("c")
    m.close(a)
    c = m.open("c")
    assert c.state_slot == a.state_slot and float(m.state[0][c.state_slot].abs().sum()) == 0.0
    m.close(b)
    m.close(c)
    m.check_invariants()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_nothing(seed):
    """Requests open, grow by random portions, and close in random order against a small pool."""
    rng = random.Random(seed)
    m = manager([FULL, WIN, WIN], page=8, pages=[24, 12], seqs=5)
    live, counter, reused = {}, 0, set()
    seen_pages = set()
    for _ in range(400):
        action = rng.random()
        if action < 0.25 and len(live) < 5:
            live[counter] = m.open(counter)
            counter += 1
        elif action < 0.85 and live:
            rid = rng.choice(list(live))
            n = rng.choice((1, 1, 1, 2, 5, 8, 17, 33))
            if m.can_reserve(live[rid], n):
                m.reserve(live[rid], n)
                for page in live[rid].held_pages(0):
                    if page in seen_pages and page not in reused:
                        reused.add(page)
                seen_pages.update(live[rid].held_pages(0))
                m.commit(live[rid], n)
            else:
                before = m.free_pages()
                with pytest.raises(OutOfPages):
                    m.reserve(live[rid], n)
                assert m.free_pages() == before
        elif live:
            rid = rng.choice(list(live))
            m.close(live.pop(rid))
        m.check_invariants()
    for s in live.values():
        m.close(s)
    assert m.free_pages() == [24, 12] and m.slots.num_free == 5
    assert reused, "the pool was never tight enough to hand a page on"

"""The cache manager: no page lost, held twice or freed twice, under random orders of requests;
atomic reservation; windows give pages back; state slots."""
import random

import pytest
import torch

from flexengine_b200.cache import RELEASED, CacheExhausted, CacheManager, PagePool
from flexengine_b200.parts.spec import CacheGroupSpec

FULL = CacheGroupSpec("attention", "full", slots=2, kv_heads=2, head_dim=4)
STATE = CacheGroupSpec("state", "state", slots=1, state_shape=(3,))
WINDOW = CacheGroupSpec("local", "window", slots=1, kv_heads=1, head_dim=4, window=10)


def manager(groups=(FULL, STATE), pages=8, page_size=4, max_requests=3):
    return CacheManager(list(groups), pages, page_size, max_requests, torch.float32, "cpu")


def test_page_pool_basics():
    pool = PagePool(4)
    a = pool.allocate(3)
    assert a == [0, 1, 2] and pool.free_pages == 1
    with pytest.raises(CacheExhausted):
        pool.allocate(2)
    assert pool.free_pages == 1                      # the failed call took nothing
    pool.retain(1)
    pool.release(1)
    assert pool.refs[1] == 1 and pool.free_pages == 1
    pool.release(1)
    assert pool.free_pages == 2
    with pytest.raises(RuntimeError, match="released more often"):
        pool.release(1)
    with pytest.raises(ValueError):
        pool.retain(3)
    assert pool.allocate(2) == [3, 1]                # first in, first out
    pool.assert_invariants({0: 1, 2: 1, 3: 1, 1: 1})
    with pytest.raises(AssertionError):
        pool.assert_invariants({0: 1})


def test_reserve_is_atomic_and_pages_come_back():
    m = manager(pages=4)
    m.reserve("a", 9)                                # 3 pages
    assert m.used_pages == 3 and m.reserved_tokens("a") == 12
    with pytest.raises(CacheExhausted):
        m.reserve("b", 5)                            # needs 2, 1 free
    assert "b" not in m.requests and m.used_pages == 3 and len(m.free_state_slots) == 2
    m.reserve("b", 4)
    with pytest.raises(CacheExhausted):
        m.reserve("a", 13)
    assert len(m.table("a", 0)) == 3
    m.commit("a", 9)
    with pytest.raises(IndexError):
        m.commit("a", 4)
    m.assert_invariants()
    m.free("a"); m.free("a")                         # freeing twice is harmless
    assert m.used_pages == 1
    m.reserve("c", 12)
    assert set(m.table("c", 0)) & set(m.table("b", 0)) == set()
    m.assert_invariants()


def test_slot_mapping_and_block_boundaries():
    m = manager(pages=6, page_size=4)
    m.reserve("a", 6)
    t = m.table("a", 0)
    assert m.slot_mapping("a", 0, 3, 3) == [t[0] * 4 + 3, t[1] * 4 + 0, t[1] * 4 + 1]
    with pytest.raises(IndexError):
        m.slot_mapping("a", 0, 6, 3)


def test_state_slots_are_assigned_zeroed_and_released():
    m = manager(max_requests=2)
    a = m.admit("a").state_slot
    m.groups[1].storage[0, a] = 7.0
    b = m.admit("b").state_slot
    assert a != b
    with pytest.raises(CacheExhausted, match="state slot"):
        m.admit("c")
    m.free("a")
    c = m.admit("c").state_slot
    assert c == a and float(m.groups[1].storage[0, c].abs().sum()) == 0.0
    m.assert_invariants()


def test_window_group_gives_back_pages_the_window_has_passed():
    # a window of 10 keys and portions of up to 7 tokens straddle at most 6 pages of 4
    m = manager(groups=(FULL, WINDOW, STATE), pages=[16, 6, 0], page_size=4)
    fed = 0
    for n in (3, 5, 4, 1, 1, 6, 2, 7, 1, 1, 1):
        m.reserve("a", fed + n)
        m.slot_mapping("a", 1, fed, n)                # the pages written now are all held
        m.commit("a", n)
        fed += n
        table = m.table("a", 1)
        first_needed = fed - 10 + 1
        for j, page in enumerate(table):
            assert (page == RELEASED) == ((j + 1) * 4 <= first_needed), (fed, j, table)
        assert m.groups[1].pool.used_pages <= 6      # 32 tokens ran through a pool of 6 pages
        m.assert_invariants()
    assert len(m.table("a", 0)) == 8 and RELEASED not in m.table("a", 0)
    m.free("a")
    assert m.groups[1].pool.free_pages == 6 and m.groups[0].pool.free_pages == 16


def test_shared_prefix_pages_are_counted_and_not_written():
    m = manager(groups=(FULL,), pages=8, page_size=4)
    m.reserve("a", 10); m.commit("a", 10)
    m.share_prefix("a", "b", 9)                       # two complete pages
    assert m.tokens_of("b") == 8 and m.table("b", 0) == m.table("a", 0)[:2]
    m.assert_invariants()
    with pytest.raises(RuntimeError, match="shared"):
        m.slot_mapping("a", 0, 4, 1)
    m.reserve("b", 12)
    assert m.slot_mapping("b", 0, 8, 2)
    m.free("a")
    assert m.used_pages == 3                          # b still holds the shared pages
    m.free("b")
    assert m.used_pages == 0
    m.assert_invariants()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_nothing(seed):
    rng = random.Random(seed)
    m = manager(groups=(FULL, WINDOW, STATE), pages=[12, 6, 0], page_size=4, max_requests=4)
    live, done, counter = {}, 0, 0
    for _ in range(400):
        action = rng.random()
        if action < 0.25 and len(live) < 4:
            rid = f"r{counter}"; counter += 1
            m.admit(rid); live[rid] = 0
        elif action < 0.8 and live:
            rid = rng.choice(list(live))
            n = rng.choice((1, 1, 2, 3, 7))
            before = {gi: list(m.table(rid, gi)) for gi, _ in m.paged}
            try:
                m.reserve(rid, live[rid] + n)
            except CacheExhausted:
                assert {gi: list(m.table(rid, gi)) for gi, _ in m.paged} == before
                victim = rng.choice(list(live))
                m.free(victim); del live[victim]; done += 1
            else:
                m.commit(rid, n); live[rid] += n
        elif live:
            rid = rng.choice(list(live))
            m.free(rid); del live[rid]; done += 1
        m.assert_invariants()
        held = [p for rc in m.requests.values() for p in rc.tables[0] if p != RELEASED]
        assert len(held) == len(set(held))
    for rid in list(live):
        m.free(rid)
    m.assert_invariants()
    assert m.groups[0].pool.free_pages == 12 and m.groups[1].pool.free_pages == 6
    assert len(m.free_state_slots) == 4 and done > 10


@pytest.mark.parametrize("seed", range(4))
def test_random_orders_with_shared_prefixes(seed):
    """Requests that start on a donor's complete pages, in random order with growth and release: a shared page is
    counted once per holder, comes back only when its last holder lets go, and is never among a holder's writable slots."""
    rng = random.Random(100 + seed)
    m = manager(groups=(FULL, STATE), pages=14, page_size=4, max_requests=5)
    live, counter, shared_seen = {}, 0, 0
    for _ in range(500):
        action = rng.random()
        if action < 0.15 and len(live) < 5:
            rid = f"r{counter}"; counter += 1
            donors = [d for d, n in live.items() if n >= 4]
            if donors and rng.random() < 0.7:
                donor = rng.choice(donors)
                tokens = rng.randrange(4, live[donor] + 1)
                m.share_prefix(donor, rid, tokens)
                live[rid] = (tokens // 4) * 4
                assert m.tokens_of(rid) == live[rid] and m.table(rid, 0) == m.table(donor, 0)[:live[rid] // 4]
                shared_seen += 1
            else:
                m.admit(rid); live[rid] = 0
        elif action < 0.8 and live:
            rid = rng.choice(list(live))
            n = rng.choice((1, 2, 5))
            try:
                m.reserve(rid, live[rid] + n)
            except CacheExhausted:
                victim = rng.choice(list(live))
                m.free(victim); del live[victim]
            else:
                # what this request may write lies past every page it shares
                slots = m.slot_mapping(rid, 0, live[rid], n)
                refs = m.groups[0].pool.refs
                assert all(refs[s // 4] == 1 for s in slots)
                m.commit(rid, n); live[rid] += n
        elif live:
            rid = rng.choice(list(live))
            m.free(rid); del live[rid]
        m.assert_invariants()
        held = set(p for rc in m.requests.values() for p in rc.tables[0])
        assert m.groups[0].pool.used_pages == len(held)
    for rid in list(live):
        m.free(rid)
    m.assert_invariants()
    assert m.used_pages == 0 and len(m.free_state_slots) == 5 and shared_seen > 5

"""The cache manager's bookkeeping (no GPU): no page lost, held twice or freed
twice, under random orders of requests; windows give pages back; state slots."""
import random

import pytest
from hypothesis import given, settings, strategies as st

from zinfer_b200.cache import CacheManager, OutOfPages, PagePool
from zinfer_b200.parts import KVCacheNeed


def test_pool_reuses_last_freed_first_and_refuses_double_free():
    pool = PagePool(4)
    a = pool.alloc(3)
    assert a == [0, 1, 2] and pool.num_free == 1
    pool.free([1])
    assert pool.alloc(1) == [1]          # the page freed last comes back first
    with pytest.raises(OutOfPages):
        pool.alloc(2)
    assert pool.num_free == 1            # a refused request takes nothing
    pool.free([0, 1])
    with pytest.raises(ValueError, match="not in use"):
        pool.free([0])
    with pytest.raises(ValueError):
        pool.free([2, 2])
    pool.check()


def _manager(num_pages=8, page=4, window=None, extra=None, max_requests=4):
    needs = {"l0": KVCacheNeed(2, 16, None), "l1": KVCacheNeed(2, 16, None)}
    if window:
        needs["w0"] = KVCacheNeed(2, 16, window)
    if extra:
        needs.update(extra)
    return CacheManager(needs, ["s0"], page, num_pages, max_requests)


def test_equal_needs_share_a_group_and_a_block_table():
    m = _manager(window=6, extra={"other": KVCacheNeed(1, 32, None)})
    assert len(m.groups) == 3
    assert m.group_of["l0"] == (0, 0) and m.group_of["l1"] == (0, 1)
    assert m.group_of["w0"][0] == 1 and m.group_of["other"][0] == 2


def test_reserve_commit_slots_and_free():
    m = _manager(num_pages=5, page=4)
    m.add_request("a")
    m.reserve("a", 6)
    assert m.block_table("a", 0) == [0, 1]
    assert m.slots_for("a", 0, 0, 6) == [0, 1, 2, 3, 4, 5]
    m.commit("a", 6)
    m.reserve("a", 1)                     # position 6 fits in the second page
    assert m.block_table("a", 0) == [0, 1]
    m.commit("a", 1)
    m.add_request("b")
    with pytest.raises(OutOfPages):
        m.reserve("b", 13)                # 4 pages wanted, 3 free
    assert m.block_table("b", 0) == [] and m.free_pages() == [3]
    m.reserve("b", 12)
    m.free_request("a")
    assert m.free_pages() == [2]
    m.add_request("c")
    m.reserve("c", 1)
    assert m.block_table("c", 0) == [1]   # a's last page, reused at once
    with pytest.raises(KeyError):
        m.free_request("a")
    with pytest.raises(KeyError):
        m.add_request("b")
    m.check()


def test_window_gives_pages_back_as_it_passes():
    m = CacheManager({"w": KVCacheNeed(1, 16, 6)}, [], 4, 5, 2)
    m.add_request("a")
    used = []
    for step in range(10):                # 3 tokens per step
        m.reserve("a", 3)
        m.commit("a", 3)
        used.append(m.groups[0].pool.num_used)
        table = m.block_table("a", 0)
        first_needed = m.length("a") - 6 + 1
        for b, page in enumerate(table):
            assert (page == -1) == ((b + 1) * 4 <= first_needed), (step, table)
    assert max(used) <= 3                 # window 6 + portion 3, pages of 4: never more than 3 live pages
    with pytest.raises(RuntimeError, match="given back"):
        m.slots_for("a", 0, 0, 1)
    m.free_request("a")
    assert m.groups[0].pool.num_used == 0
    m.check()


def test_state_slots_are_reused_and_limited():
    m = _manager(max_requests=2)
    a, b = m.add_request("a"), m.add_request("b")
    assert {a.state_slot, b.state_slot} == {0, 1}
    with pytest.raises(OutOfPages):
        m.add_request("c")
    m.free_request("a")
    assert m.add_request("c").state_slot == a.state_slot
    m.check()


@settings(max_examples=60, deadline=None)
@given(st.integers(0, 2 ** 32 - 1), st.integers(3, 24), st.sampled_from([1, 4, 16]), st.sampled_from([None, 5, 17]))
def test_random_orders_never_lose_or_duplicate_a_page(seed, num_pages, page, window):
    rng = random.Random(seed)
    needs = {"full": KVCacheNeed(1, 16, None)}
    if window:
        needs["win"] = KVCacheNeed(1, 16, window)
    m = CacheManager(needs, ["s"], page, num_pages, 4)
    live, next_id = [], 0
    for _ in range(120):
        op = rng.random()
        if op < 0.3 and len(live) < 4:
            m.add_request(next_id)
            live.append(next_id)
            next_id += 1
        elif op < 0.85 and live:
            rid = rng.choice(live)
            n = rng.randint(1, 2 * page + 3)
            before = m.free_pages()
            if m.can_reserve(rid, n):
                m.reserve(rid, n)
                for gi in range(len(m.groups)):
                    slots = m.slots_for(rid, gi, m.length(rid), n)
                    assert len(set(slots)) == n
                m.commit(rid, n)
            else:
                with pytest.raises(OutOfPages):
                    m.reserve(rid, n)
                assert m.free_pages() == before
        elif live:
            rid = live.pop(rng.randrange(len(live)))
            m.free_request(rid)
        m.check()
    for rid in live:
        m.free_request(rid)
    m.check()
    assert all(g.pool.num_used == 0 for g in m.groups) and m.slots.num_used == 0

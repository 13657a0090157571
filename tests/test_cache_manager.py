"""The cache manager's bookkeeping, without a GPU: no page is lost, held twice or freed twice."""
import random

import pytest

from vllm_cpp_b200.cache.block_pool import BlockPool, PageError
from vllm_cpp_b200.cache.manager import RELEASED, CacheManager, OutOfPages
from vllm_cpp_b200.parts.base import PagedKVSpec, StateSpec

FULL = PagedKVSpec(2, 16, 0)
WIN = PagedKVSpec(2, 16, 24)


def test_pool_counts_like_the_reference():
    # tests/unit/test_block_manager.cpp:4-26 of the reference
    p = BlockPool(4)
    a, b = p.acquire(), p.acquire()
    assert p.num_free == 2 and p.can_allocate(2) and not p.can_allocate(3)
    p.inc_ref(a)
    assert not p.release(a) and p.num_free == 2
    assert p.release(a) and p.num_free == 3
    with pytest.raises(PageError):
        p.release(a)
    with pytest.raises(PageError):
        p.release(99)
    assert p.acquire() == a          # the page just given back is handed out next
    with pytest.raises(ValueError):
        BlockPool(0)


def check_invariants(m: CacheManager):
    for gi, g in enumerate(m.paged):
        held = []
        for rc in m.requests.values():
            held += [b for b in rc.tables[gi] if b != RELEASED]
        assert len(held) == len(set(held)), "a page is held twice"
        free = g.pool._free
        assert len(free) == len(set(free)), "a page is in the free list twice"
        assert not set(free) & set(held), "a held page is in the free list"
        assert len(free) + len(held) == m.num_pages, "a page is lost"
        assert all(g.pool.ref_count(b) == 1 for b in held)
    slots = [rc.slot for rc in m.requests.values()]
    assert len(slots) == len(set(slots)) and len(slots) + len(m._free_slots) == m.max_num_seqs
    # the tables as rows of one array (what the step function copies) say the same as the lists
    for gi in range(len(m.paged)):
        width = 1 + max([len(rc.tables[gi]) for rc in m.requests.values()] + [3])
        rows = m.table_rows(gi, width if len(m.requests) % 2 else width + 2)      # widened now and then
        for rc in m.requests.values():
            t = rc.tables[gi]
            assert list(rows[rc.slot, : len(t)]) == t and (rows[rc.slot, len(t):] == RELEASED).all()


def test_groups_follow_the_layers_needs():
    m = CacheManager([FULL, WIN, FULL, StateSpec((4,)), None, WIN], 16, 10, 4)
    assert [g.layers for g in m.paged] == [[0, 2], [1, 5]]
    assert [g.layers for g in m.state] == [[3]]
    v = m.views()
    assert v[4] is None and v[0].group == 0 and v[1].group == 1 and v[5].group == 1


def test_reserve_commit_free():
    m = CacheManager([FULL], 16, 4, 2)
    m.add_request("a")
    assert m.pages_needed("a", 17) == [2]
    m.reserve("a", 17)
    m.commit("a", 17)
    assert m.table("a", 0) == [0, 1] and m.num_tokens("a") == 17
    assert m.pages_needed("a", 15) == [0] and m.pages_needed("a", 16) == [1]
    m.add_request("b")
    assert m.can_append("b", 32) and not m.can_append("b", 33)
    with pytest.raises(OutOfPages):
        m.reserve("b", 33)
    assert m.table("b", 0) == [] and m.num_free_pages() == 2          # all or nothing
    with pytest.raises(OutOfPages):
        m.add_request("c")                                            # no slot left
    m.free_request("a")
    assert m.num_free_pages() == 4
    m.reserve("b", 33)
    assert m.table("b", 0)[0] == 0                                    # a's first page is used again first
    check_invariants(m)
    with pytest.raises(KeyError):
        m.free_request("a")


def test_window_pages_come_back_when_the_window_has_passed():
    m = CacheManager([FULL, WIN], 16, 8, 2)
    m.add_request("a")
    for n in (40, 1, 1, 30, 9):
        m.reserve("a", n)
        m.commit("a", n)
        check_invariants(m)
    total = 81
    assert m.num_tokens("a") == total
    full, win = m.table("a", 0), m.table("a", 1)
    assert RELEASED not in full and len(full) == 6
    # keys at or below total - 24 = 57 are never read again: pages 0..2 hold positions 0..47
    assert win[:3] == [RELEASED] * 3 and RELEASED not in win[3:]
    assert m.paged[1].pool.num_free == 8 - 3 and m.paged[0].pool.num_free == 2
    assert m.max_appendable("a") == 2 * 16 + (6 * 16 - total)
    m.free_request("a")
    assert m.num_free_pages() == 8
    check_invariants(m)


def test_state_slot_for_every_request_even_without_state():
    m = CacheManager([FULL], 16, 8, 3)
    assert [m.add_request(i).slot for i in range(3)] == [0, 1, 2]
    m.free_request(1)
    assert m.add_request("x").slot == 1


@pytest.mark.parametrize("seed", range(5))
def test_random_orders_keep_every_page_accounted_for(seed):
    rng = random.Random(seed)
    m = CacheManager([FULL, WIN, FULL], 16, 24, 5)
    live = {}
    for step in range(600):
        op = rng.random()
        if op < 0.25 and m.has_free_slot():
            rid = f"r{step}"
            m.add_request(rid)
            live[rid] = 0
        elif op < 0.85 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 7, 16, 33])
            if m.can_append(rid, n):
                m.reserve(rid, n)
                if rng.random() < 0.9:          # sometimes a reservation is left uncommitted
                    m.commit(rid, n)
                    live[rid] += n
            else:
                with pytest.raises(OutOfPages):
                    m.reserve(rid, n)
        elif live:
            rid = rng.choice(list(live))
            m.free_request(rid)
            del live[rid]
        check_invariants(m)
        for rid, n in live.items():
            assert m.num_tokens(rid) == n
    for rid in list(live):
        m.free_request(rid)
    check_invariants(m)
    assert all(g.pool.num_free == 24 for g in m.paged)

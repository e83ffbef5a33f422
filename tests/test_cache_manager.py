"""The cache manager: no page lost, held twice or freed twice, under random orders of requests."""
import random

import pytest

from inferrs_b200.cache.manager import RELEASED, CacheError, CacheManager, GroupLayout, OutOfPages, PagePool


def test_pool_is_fifo_and_refuses_double_free():
    p = PagePool(4)
    assert p.take(3) == [0, 1, 2]
    p.give_back([1])
    assert p.take(2) == [3, 1]          # freed pages go to the back (kv_cache.rs:128-139)
    with pytest.raises(OutOfPages):
        p.take(2)
    p.give_back([0])
    with pytest.raises(CacheError, match="twice"):
        p.give_back([0])
    with pytest.raises(CacheError, match="outside"):
        p.give_back([9])


def test_reserve_is_all_or_nothing():
    m = CacheManager([GroupLayout("full")], page_size=4, n_pages=[5], max_requests=3)
    m.admit("a"); m.admit("b")
    m.reserve({"a": 9})                  # 3 pages
    m.commit("a", 9)
    with pytest.raises(OutOfPages):
        m.reserve({"a": 3, "b": 9})      # 0 + 3 pages > 2 free... a needs 0 more, b needs 3
    assert m.pools[0].n_free == 2 and m.block_table("b", 0) == []
    m.reserve({"a": 3, "b": 8})
    assert m.pools[0].n_free == 0
    m.check_invariants()
    m.release("a")
    assert m.pools[0].n_free == 3
    with pytest.raises(CacheError, match="not live"):
        m.release("a")
    m.check_invariants()


def test_slots_run_out_and_come_back():
    m = CacheManager([GroupLayout("full")], page_size=4, n_pages=[8], max_requests=2)
    s0, s1 = m.admit(0), m.admit(1)
    assert {s0, s1} == {0, 1}
    with pytest.raises(OutOfPages, match="slot"):
        m.admit(2)
    with pytest.raises(CacheError, match="already live"):
        m.admit(1)
    m.release(0)
    assert m.admit(2) == s0


def test_window_group_gives_pages_back_when_the_window_has_passed():
    m = CacheManager([GroupLayout("full"), GroupLayout("win", window=6)], page_size=4, n_pages=[16, 16], max_requests=2)
    m.admit("r")
    held = 0
    for n in [5, 1, 1, 9, 1, 1, 1, 2]:
        m.reserve({"r": n})
        # every key that this step's queries may see is still there: positions held-5 .. held+n-1
        t = m.block_table("r", 1)
        for pos in range(max(0, held - 5), held + n):
            assert t[pos // 4] != RELEASED
        m.commit("r", n)
        held += n
        first_needed = held - 6 + 1
        for i, p in enumerate(m.block_table("r", 1)):
            assert (p == RELEASED) == ((i + 1) * 4 <= first_needed), (held, i)
        assert all(p != RELEASED for p in m.block_table("r", 0))
        m.check_invariants()
    live_win = sum(p != RELEASED for p in m.block_table("r", 1))
    assert live_win <= 3 and m.pools[1].n_free == 16 - live_win
    m.release("r")
    assert m.pools[0].n_free == 16 and m.pools[1].n_free == 16


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_never_lose_a_page(seed):
    rng = random.Random(seed)
    groups = [GroupLayout("full"), GroupLayout("win", window=rng.choice([3, 7, 20]))]
    m = CacheManager(groups, page_size=rng.choice([1, 4, 16]), n_pages=[rng.randint(6, 40), rng.randint(6, 40)],
                     max_requests=4)
    live, next_id = {}, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 4:
            m.admit(next_id); live[next_id] = 0; next_id += 1
        elif op < 0.4 and live:
            rid = rng.choice(list(live)); m.release(rid); del live[rid]
        elif live:
            chosen = rng.sample(list(live), rng.randint(1, len(live)))
            wants = {rid: rng.randint(1, 24) for rid in chosen}
            before = [p.n_free for p in m.pools]
            try:
                m.reserve(wants)
            except OutOfPages:
                assert [p.n_free for p in m.pools] == before
            else:
                for rid, n in wants.items():
                    m.commit(rid, n); live[rid] += n
                    assert m.n_tokens(rid) == live[rid]
        m.check_invariants()
    for rid in list(live):
        m.release(rid)
    assert [p.n_free for p in m.pools] == [p.n_pages for p in m.pools] and m.n_free_slots == 4

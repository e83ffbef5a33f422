"""The cache manager (native code behind a Python front): no page lost, held twice or freed twice, under
random orders of requests, and every answer equal to the plain model's."""
import random

import pytest

import plain_cache
from inferrs_b200.cache.manager import RELEASED, CacheError, CacheManager, GroupLayout, OutOfPages


def test_the_plain_models_pool_is_fifo_and_refuses_double_free():
    p = plain_cache.PagePool(4)
    assert p.take(3) == [0, 1, 2]
    p.give_back([1])
    assert p.take(2) == [3, 1]          # freed pages go to the back (kv_cache.rs:128-139)
    with pytest.raises(plain_cache.OutOfPages):
        p.take(2)
    p.give_back([0])
    with pytest.raises(plain_cache.CacheError, match="twice"):
        p.give_back([0])
    with pytest.raises(plain_cache.CacheError, match="outside"):
        p.give_back([9])


def test_pages_come_back_in_the_order_they_were_freed():
    """The native pool is first in, first out as the reference's is (kv_cache.rs:104-139): tables show it."""
    m = CacheManager([GroupLayout("full")], page_size=1, n_pages=[4], max_requests=2)
    m.admit("a")
    m.reserve({"a": 3}); m.commit("a", 3)
    assert m.block_table("a", 0) == [0, 1, 2]
    m.release("a")
    m.admit("b")
    m.reserve({"b": 3}); m.commit("b", 3)
    assert m.block_table("b", 0) == [3, 0, 1]


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


@pytest.mark.parametrize("seed", range(8))
def test_native_manager_answers_as_the_plain_model_does(seed):
    """The same random calls go to the native manager and to the plain model: free pages, slots, token counts,
    block tables (so also the order in which pages are used again) and refusals must agree after every call."""
    rng = random.Random(100 + seed)
    windows = [None, rng.choice([2, 5, 9, 33])] if seed % 2 else [rng.choice([4, 17]), None, None]
    page_size = rng.choice([1, 3, 16])
    n_pages = [rng.randint(5, 30) for _ in windows]
    nat = CacheManager([GroupLayout(f"g{i}", w) for i, w in enumerate(windows)], page_size, n_pages, max_requests=5)
    ref = plain_cache.CacheManager([plain_cache.GroupLayout(f"g{i}", w) for i, w in enumerate(windows)], page_size,
                                   n_pages, max_requests=5)
    live, next_id = [], 0
    for _ in range(500):
        op = rng.random()
        if op < 0.2:
            rid = ("r", next_id)
            next_id += 1
            if len(live) < 5:
                assert nat.admit(rid) == ref.admit(rid)
                live.append(rid)
            else:
                with pytest.raises(OutOfPages):
                    nat.admit(rid)
                with pytest.raises(plain_cache.OutOfPages):
                    ref.admit(rid)
        elif op < 0.35 and live:
            rid = live.pop(rng.randrange(len(live)))
            nat.release(rid)
            ref.release(rid)
        elif live:
            wants = {rid: rng.randint(1, 20) for rid in rng.sample(live, rng.randint(1, len(live)))}
            assert nat.can_reserve(wants) == ref.can_reserve(wants)
            for rid, n in wants.items():
                assert nat.pages_needed(rid, n) == ref.pages_needed(rid, n)
            free_a = [max(0, p.n_free - rng.randint(0, 6)) for p in nat.pools]
            free_b = list(free_a)
            assert nat.fit_in_order(list(wants), list(wants.values()), free_a) == \
                ref.fit_in_order(list(wants), list(wants.values()), free_b) and free_a == free_b
            try:
                ref.reserve(wants)
            except plain_cache.OutOfPages:
                with pytest.raises(OutOfPages):
                    nat.reserve(wants)
            else:
                nat.reserve(wants)
                for rid, n in wants.items():
                    k = rng.randint(1, n)           # a step may write fewer tokens than were reserved
                    nat.commit(rid, k)
                    ref.commit(rid, k)
        assert [p.n_free for p in nat.pools] == [p.n_free for p in ref.pools]
        assert nat.n_free_slots == ref.n_free_slots and nat.n_live == ref.n_live
        for rid in live:
            assert nat.n_tokens(rid) == ref.n_tokens(rid) and nat.slot(rid) == ref.slot(rid)
            for g in range(len(windows)):
                assert nat.block_table(rid, g) == ref.block_table(rid, g)
        nat.check_invariants()
        ref.check_invariants()
    with pytest.raises(CacheError, match="not live"):
        nat.n_tokens(("r", -1))


@pytest.mark.parametrize("seed", range(4))
def test_native_description_of_a_decode_step_equals_the_general_builders(seed):
    """Token ids, positions, lengths, slots and block tables of a step of single tokens, padded to a bucket, as
    native code lays them out, against the general builder (which the step function uses for every other step)."""
    import numpy as np
    import torch
    from inferrs_b200.engine.batch import StepEntry, build_context
    rng = random.Random(seed)
    windows = [None, 11] if seed % 2 else [None]
    m = CacheManager([GroupLayout(f"g{i}", w) for i, w in enumerate(windows)], page_size=4,
                     n_pages=[160] * len(windows), max_requests=6)
    vocab, max_pos, bucket = 1000, 200, 8
    fixed = [(max_pos + 3) // 4] * len(windows)
    live = []
    for i in range(5):
        m.admit(i)
        n = rng.randint(1, 60)
        m.reserve({i: n}); m.commit(i, n)
        live.append(i)
    for _ in range(40):
        chosen = rng.sample(live, rng.randint(1, len(live)))
        m.reserve({rid: 1 for rid in chosen})
        tokens = [rng.randrange(vocab) for _ in chosen]
        out = np.full(4096, 12345, dtype=np.int32)
        code, _ = m.describe_decode(chosen, tokens, bucket, fixed, vocab, max_pos, out.ctypes.data, out.size)
        ctx = build_context([StepEntry(rid, [t], [0]) for rid, t in zip(chosen, tokens)], m, None, vocab, max_pos,
                            torch.device("cpu"), fixed_pages=fixed, pad_to=bucket)
        host = ctx.extra["host"]
        assert code == host.size and np.array_equal(out[:code], host)
        for rid in chosen:
            m.commit(rid, 1)
    # refusals: a token outside the vocabulary, a request that is full, a request that is not live
    m.reserve({0: 1})
    out = np.zeros(4096, dtype=np.int32)
    assert m.describe_decode([0], [vocab], bucket, fixed, vocab, max_pos, out.ctypes.data, out.size)[0] < 0
    assert m.describe_decode([0], [1], bucket, fixed, vocab, m.n_tokens(0), out.ctypes.data, out.size)[0] < 0
    with pytest.raises(CacheError, match="not live"):
        m.describe_decode([99], [1], bucket, fixed, vocab, max_pos, out.ctypes.data, out.size)


@pytest.mark.parametrize("seed", range(4))
def test_native_description_of_a_padded_step_equals_the_general_builders(seed):
    """Steps of any portions, padded to a fixed shape with tile lists of fixed length: native code against the
    general builder, number for number."""
    import numpy as np
    import torch
    from inferrs_b200.engine.batch import StepEntry, build_context
    rng = random.Random(50 + seed)
    windows = [None, 13] if seed % 2 else [None]
    m = CacheManager([GroupLayout(f"g{i}", w) for i, w in enumerate(windows)], page_size=4,
                     n_pages=[400] * len(windows), max_requests=6)
    vocab, max_pos = 1000, 300
    fixed = [(max_pos + 3) // 4] * len(windows)
    tile_sizes = [(32, True), (16, False)] if seed < 2 else [(64, True)]
    live = list(range(5))
    for i in live:
        m.admit(i)
    for _ in range(40):
        chosen = rng.sample(live, rng.randint(1, len(live)))
        counts = [rng.choice([1, 1, 2, 7, 33]) for _ in chosen]
        if any(m.n_tokens(rid) + n > max_pos for rid, n in zip(chosen, counts)):
            break
        m.reserve(dict(zip(chosen, counts)))
        tokens = [[rng.randrange(vocab) for _ in range(n)] for n in counts]
        wants = [sorted(rng.sample(range(n), rng.randint(0, min(n, 3)))) for n in counts]
        rows = 64 if sum(counts) <= 64 else 256
        out = np.full(8192, 12345, dtype=np.int32)
        # room in the tile lists for as many requests as the step has, for one more, or for every request
        tile_pad = rng.choice([len(chosen), len(chosen) + 1, 7])
        code, _ = m.describe_step(chosen, tokens, wants, rows, 7, 20, fixed, tile_sizes, tile_pad, vocab, max_pos,
                                  out.ctypes.data, out.size)
        ctx = build_context([StepEntry(rid, t, w) for rid, t, w in zip(chosen, tokens, wants)], m, None, vocab, max_pos,
                            torch.device("cpu"), fixed_pages=fixed, pad_rows=rows, pad_requests=7, pad_wanted=20,
                            tile_sizes=tile_sizes, tile_pad=tile_pad)
        host = ctx.extra["host"]
        assert code == host.size, (code, host.size)
        assert np.array_equal(out[:code], host)
        # the tiles stand at the end of their list, the one that sees the fewest keys first
        for (tpt, portions_only) in tile_sizes:
            req, row0, n_tiles = ctx.attention_tiles(tpt, portions_only)
            req, row0 = req.tolist(), row0.tolist()
            real = [k for k in range(n_tiles) if req[k] >= 0]
            assert real == list(range(n_tiles - len(real), n_tiles))
            last = [ctx.positions[min(row0[k] + tpt, ctx.q_start[req[k] + 1]) - 1].item() for k in real]
            assert last == sorted(last)
            want_tiles = sum((n + tpt - 1) // tpt for n in counts if not (portions_only and n == 1))
            assert len(real) == want_tiles
        for rid, n in zip(chosen, counts):
            m.commit(rid, n)
    m.reserve({0: 2})
    out = np.zeros(8192, dtype=np.int32)
    assert m.describe_step([0], [[1, vocab]], [[0]], 64, 7, 20, fixed, tile_sizes, 7, vocab, max_pos, out.ctypes.data, out.size)[0] < 0
    assert m.describe_step([0], [[1, 2]], [[2]], 64, 7, 20, fixed, tile_sizes, 7, vocab, max_pos, out.ctypes.data, out.size)[0] < 0
    # more requests with tiles than the lists have room for beyond rows / tokens: refused by both
    m.reserve({1: 2, 2: 2})
    many = ([0, 1, 2], [[1, 2], [3, 4], [5, 6]], [[0], [0], [0]])
    if all(po for _, po in tile_sizes):
        assert m.describe_step(*many, 64, 7, 20, fixed, tile_sizes, 0, vocab, max_pos, out.ctypes.data, out.size)[0] < 0

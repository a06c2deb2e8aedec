"""The cache manager on the host: no page lost, held twice or freed twice, under
random orders of requests; windows give pages back; slots for fixed state (no GPU).
Every test runs on the Python implementation and on the C++ core."""
import random

import pytest

from vllm_lite_b200.cache import CacheLayout, CacheManager, FixedState, OutOfPages, PagedKV, Pool, PoolError
from vllm_lite_b200.cache.native import NativeCacheManager


@pytest.fixture(params=["python", "native"])
def make(request):
    """Both implementations of the bookkeeping: the Python reference and the C++ core."""
    return CacheManager if request.param == "python" else NativeCacheManager


def layout(*needs, cache_of=None):
    return CacheLayout.from_needs(list(needs), cache_of or [None] * len(needs))


def test_pool_hands_out_each_unit_once_and_reuses_lifo():
    p = Pool(4)
    a = p.allocate(3)
    assert a == [0, 1, 2] and p.allocate(2) is None and p.free_count == 1
    p.release([1])
    assert p.allocate(1) == [1]                      # most recently freed first
    p.release([0, 2])
    assert p.allocate(2) == [0, 2]
    p.check()


def test_pool_refuses_double_free_and_foreign_units():
    p = Pool(3)
    got = p.allocate(2)
    p.release(got)
    with pytest.raises(PoolError):
        p.release([got[0]])
    with pytest.raises(PoolError):
        p.release([7])
    with pytest.raises(PoolError):
        p.release([2])                               # never handed out


def test_layers_with_equal_needs_share_a_group_others_get_their_own():
    full, win, state = PagedKV(2, 16), PagedKV(2, 16, window=32), FixedState((4, 8))
    lay = layout(full, win, full, state, None, win, cache_of=[None, None, None, None, None, None])
    assert lay.paged_groups == [full, win] and lay.paged_members == [[0, 2], [1, 5]]
    assert lay.state_groups == [state] and lay.state_members == [[3]]
    assert lay.call_place[4] is None and lay.call_place[5] == ("paged", 1, 1, True)
    shared = layout(full, None, cache_of=[None, 0])
    assert shared.call_place[1] == ("paged", 0, 0, False)


def test_pages_are_taken_when_written_and_returned_at_the_end(make):
    m = make(layout(PagedKV(2, 16)), page_size=8, num_pages=6, max_requests=2)
    m.admit("a")
    assert m.append("a", 5) == 0 and m.requests["a"].block_tables == [[0]]
    assert m.append("a", 3) == 5 and m.requests["a"].block_tables == [[0]]      # still the first page
    assert m.append("a", 1) == 8 and m.requests["a"].block_tables == [[0, 1]]
    assert m.slot_of("a", 0, 9) == 1 * 8 + 1
    m.admit("b")
    assert m.pages_needed("b", 33) == [5] and not m.can_append("b", 33)
    with pytest.raises(OutOfPages):
        m.append("b", 33)
    assert m.requests["b"].block_tables == [[]] and m.free_pages() == [4]       # nothing was taken
    m.append("b", 32)
    with pytest.raises(OutOfPages):
        m.admit("c")                                                           # both slots are held
    m.free("a")
    assert m.free_pages() == [2]
    m.admit("c")
    m.append("c", 16)
    assert sorted(m.requests["c"].block_tables[0]) == [0, 1]                    # a's pages are used again
    m.check_invariants()
    with pytest.raises(KeyError):
        m.free("a")


def test_window_gives_pages_back_once_it_has_passed_them(make):
    m = make(layout(PagedKV(1, 16), PagedKV(1, 16, window=10)), page_size=4, num_pages=[16, 5], max_requests=1)
    m.admit("r")
    m.append("r", 9)
    assert m.release_behind_window("r") == 0          # next query at 9 reads 0..9
    m.append("r", 4)                                  # 13 tokens; next query at 13 reads 4..13
    assert m.release_behind_window("r") == 1
    full, win = m.requests["r"].block_tables
    assert full == [0, 1, 2, 3] and win == [-1, 1, 2, 3]
    with pytest.raises(PoolError):
        m.slot_of("r", 1, 2)
    for _ in range(30):                               # the windowed group never needs more than its 5 pages
        m.append("r", 1)
        m.release_behind_window("r")
        m.check_invariants()
    assert m.requests["r"].num_tokens == 43
    assert sum(p >= 0 for p in m.requests["r"].block_tables[1]) <= 4
    m.free("r")
    assert m.free_pages() == [16, 5]


def test_growth_is_all_groups_or_none(make):
    m = make(layout(PagedKV(1, 16), PagedKV(2, 32)), page_size=4, num_pages=[8, 2], max_requests=1)
    m.admit("r")
    m.append("r", 8)
    with pytest.raises(OutOfPages):
        m.append("r", 1)                               # the second group is full
    assert m.free_pages() == [6, 0] and m.requests["r"].num_tokens == 8


def test_state_slots_are_fresh_once(make):
    m = make(layout(FixedState((3,))), page_size=16, num_pages=0, max_requests=2)
    a, b = m.admit("a"), m.admit("b")
    assert {a.state_slot, b.state_slot} == {0, 1} and sorted(m.take_fresh_slots()) == [0, 1]
    assert m.take_fresh_slots() == []
    m.free("a")
    assert m.admit("c").state_slot == a.state_slot and m.take_fresh_slots() == [a.state_slot]


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_keep_the_books(make, seed):
    rng = random.Random(seed)
    m = make(layout(PagedKV(2, 16), PagedKV(2, 16, window=24)), page_size=8, num_pages=[40, 14], max_requests=5)
    live, n = {}, 0
    for _ in range(600):
        roll = rng.random()
        if roll < 0.2 and len(live) < 5:
            n += 1
            m.admit(n)
            live[n] = 0
        elif roll < 0.85 and live:
            rid = rng.choice(list(live))
            count = rng.choice([1, 1, 1, 2, 5, 9, 17])
            if m.can_append(rid, count):
                assert m.append(rid, count) == live[rid]
                live[rid] += count
                m.release_behind_window(rid)
            else:
                before = (m.free_pages(), [list(t) for t in m.requests[rid].block_tables])
                with pytest.raises(OutOfPages):
                    m.append(rid, count)
                assert before == (m.free_pages(), m.requests[rid].block_tables)
        elif live:
            rid = rng.choice(list(live))
            m.free(rid)
            del live[rid]
        m.check_invariants()
        for rid, tokens in live.items():
            rc = m.requests[rid]
            assert rc.num_tokens == tokens
            assert len(rc.block_tables[0]) == -(-tokens // 8)
            # every position a later query can still read has a page
            for pos in range(max(0, tokens - 24 + 1), tokens):
                assert rc.block_tables[1][pos // 8] >= 0
    for rid in list(live):
        m.free(rid)
    assert m.free_pages() == [40, 14] and m.slots.free_count == 5


def test_native_decode_step_equals_its_parts():
    """The one-call decode step of the C++ core (check, appends, packed batch, windows) leaves the
    same books and writes the same words as the calls it stands for; a step that does not fit, or
    that would take a request beyond the limit, changes nothing."""
    import numpy as np
    lay = layout(PagedKV(1, 16), PagedKV(1, 16, window=6))
    a = NativeCacheManager(lay, page_size=4, num_pages=[12, 9], max_requests=4)
    b = NativeCacheManager(lay, page_size=4, num_pages=[12, 9], max_requests=4)
    for m in (a, b):
        for rid, n in (("x", 7), ("y", 3), ("z", 12)):
            m.admit(rid)
            m.append(rid, n)
            m.release_behind_window(rid)
    ids, toks = ["z", "x", "y"], [5, 6, 7]
    for step in range(5):
        out_a = np.full(4096, 77, dtype=np.int32)
        used, off, sizes, starts = a.decode_step(ids, toks, 4, 8, 1000, out_a)
        st = [b.append(r, 1) for r in ids]
        out_b = np.full(4096, 77, dtype=np.int32)
        used_b, off_b, sizes_b, _ = b.pack_step(ids, [1, 1, 1], st, toks, [0, 1, 2, 3], [0, 0, 0], 4, 0, 8, out_b)
        for r in ids:
            b.release_behind_window(r)
        assert used == used_b and list(off) == list(off_b) and list(sizes) == list(sizes_b) and list(starts) == st
        assert (out_a[:used] == out_b[:used]).all() and (out_a[used:] == 77).all()
        for r in ids:
            assert a.requests[r].block_tables == b.requests[r].block_tables and a.requests[r].num_tokens == b.requests[r].num_tokens
        assert a.free_pages() == b.free_pages()
        a.check_invariants()
    before = (a.free_pages(), [a.requests[r].num_tokens for r in ids])
    assert a.decode_step(ids, toks, 4, 8, a.requests["z"].num_tokens, np.zeros(4096, dtype=np.int32)) is None   # z at its limit
    assert a.decode_step(ids, toks, 4, 8, 1000, np.zeros(8, dtype=np.int32))[0] < 0                             # buffer too small
    small = NativeCacheManager(lay, page_size=4, num_pages=[2, 9], max_requests=2)
    small.admit("p"); small.append("p", 4); small.admit("q"); small.append("q", 4)
    with pytest.raises(OutOfPages):
        small.decode_step(["p", "q"], [1, 2], 2, 8, 1000, np.zeros(4096, dtype=np.int32))
    assert small.free_pages() == [0, 7] and small.requests["p"].num_tokens == 4
    assert before == (a.free_pages(), [a.requests[r].num_tokens for r in ids])

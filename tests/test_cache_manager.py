"""The cache manager on the host: no page lost, held twice or freed twice, under random orders."""
import random

import pytest

from hi_b200.cache import FREED, CacheManager, OutOfPages, OutOfSlots, PagePool
from hi_b200.parts.spec import CacheSpec

GLOBAL = CacheSpec(kv_heads=2, head_dim=16, window=None)
CHUNK = CacheSpec(kv_heads=2, head_dim=16, window=("chunk", 10))
SLIDE = CacheSpec(kv_heads=2, head_dim=16, window=("sliding", 6))


def test_pool_allocate_exhaust_free_reuse():
    pool = PagePool(3)
    a, b, c = pool.take("x"), pool.take("x"), pool.take("y")
    assert sorted((a, b, c)) == [0, 1, 2] and pool.free == 0 and pool.peak_used == 3
    with pytest.raises(OutOfPages):
        pool.take("z")
    assert pool.failed_allocations == 1
    pool.give(b, "x")
    with pytest.raises(RuntimeError, match="freed twice"):
        pool.give(b, "x")
    with pytest.raises(RuntimeError, match="held by"):
        pool.give(c, "x")
    assert pool.take("z") == b and pool.owner(b) == "z"


def test_windows_give_pages_back_as_they_pass():
    m = CacheManager([GLOBAL, CHUNK, SLIDE], [16, 16, 16], page_size=4, max_requests=2)
    m.open("r")
    for step, n in enumerate([3, 9, 1, 1, 12, 2, 7]):
        m.reserve("r", n)
        m.commit("r", n)
        m.check_invariants()
        length = m.length("r")
        tg, tc, ts = (m.table(g, "r") for g in range(3))
        assert all(p != FREED for p in tg) and len(tg) == -(-length // 4)
        first_chunk = (length // 10) * 10 // 4
        assert all((p == FREED) == (b < first_chunk) for b, p in enumerate(tc)), (length, tc)
        first_slide = max(0, length - 6 + 1) // 4
        assert all((p == FREED) == (b < first_slide) for b, p in enumerate(ts)), (length, ts)
    assert m.held_pages("r")[0] == 9 and m.held_pages("r")[1] <= 3 and m.held_pages("r")[2] <= 3
    m.close("r")
    assert all(p.free == p.total for p in m.pools) and m.free_slots == 2


def test_a_portion_that_straddles_a_chunk_edge_keeps_both_chunks_for_the_step():
    m = CacheManager([CHUNK], [8], page_size=4, max_requests=1)
    m.open("r")
    m.reserve("r", 8); m.commit("r", 8)            # positions 0..7, chunk 0
    m.reserve("r", 7)                                # positions 8..14: 8, 9 read chunk 0; 10.. read chunk 1
    assert all(p != FREED for p in m.table(0, "r")) and len(m.table(0, "r")) == 4
    m.commit("r", 7)                                 # next token is 15: chunk 1 starts at 10 -> blocks 0, 1 dead
    assert [p == FREED for p in m.table(0, "r")] == [True, True, False, False]


def test_reserve_is_all_or_nothing_and_exhaustion_is_structured():
    m = CacheManager([GLOBAL, CHUNK], [4, 3], page_size=4, max_requests=2)
    m.open("a")
    m.reserve("a", 8); m.commit("a", 8)
    before = (m.pools[0].free, m.pools[1].free)
    with pytest.raises(OutOfPages) as e:
        m.reserve("a", 8)                            # global would fit (2 pages), the chunk group would not
    assert e.value.group == 1 and "insufficient_gpu_memory" in str(e.value)
    assert (m.pools[0].free, m.pools[1].free) == before
    m.check_invariants()
    assert m.pages_needed("a", 1) == [1, 1] and m.can_reserve("a", 1) and not m.can_reserve("a", 8)
    with pytest.raises(KeyError):
        m.open("a")
    m.open("b")
    with pytest.raises(OutOfSlots):
        m.open("c")


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_every_invariant(seed):
    rng = random.Random(seed)
    page = rng.choice([1, 2, 4, 8])
    m = CacheManager([GLOBAL, CHUNK, SLIDE], [rng.randint(6, 30) for _ in range(3)], page_size=page, max_requests=4)
    live, next_id, reused = {}, 0, set()
    handed = [set(), set(), set()]
    for _ in range(600):
        move = rng.random()
        if move < 0.15 and m.free_slots:
            m.open(next_id); live[next_id] = 0; next_id += 1
        elif move < 0.25 and live:
            rid = rng.choice(list(live)); m.close(rid); del live[rid]
        elif live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 3, 5, 9, 17])
            before = [list(t) for t in m.requests[rid].tables]
            try:
                m.reserve(rid, n)
            except OutOfPages:
                assert [list(t) for t in m.requests[rid].tables] == before, "a failed reserve left pages behind"
                m.close(rid); del live[rid]          # what a scheduler would do at the latest: give up the request
            else:
                for g, t in enumerate(m.requests[rid].tables):
                    for p in t[len(before[g]):]:
                        if p != FREED:
                            if p in handed[g]:
                                reused.add(g)
                            handed[g].add(p)
                m.commit(rid, n); live[rid] += n
                assert m.length(rid) == live[rid]
        m.check_invariants()
    for rid in list(live):
        m.close(rid)
    m.check_invariants()
    assert all(p.free == p.total for p in m.pools) and m.free_slots == 4
    assert reused, "no page was ever used again: the test did not stress the pools"

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


def test_step_inputs_are_packed_from_the_tables():
    """The native packing of a step's integer inputs: tokens, positions from the requests'
    lengths, sequence ids, cumulative counts, slots, wanted rows, block tables padded with -1;
    and rows of a buffer that lives on are rewritten only when their request or its tables changed."""
    import numpy as np

    m = CacheManager([GLOBAL, CHUNK], [16, 16], page_size=4, max_requests=3)
    m.open("a"); m.reserve("a", 9); m.commit("a", 9)          # a: 9 tokens in the cache
    m.open("b")
    m.reserve("a", 1); m.reserve("b", 6)                      # this step: a decodes, b brings 6 prompt tokens
    handles = m.handles_of(["a", "b"])
    widths = m.step_widths(handles)
    assert widths == [3, 3]
    n_new = np.array([1, 6], dtype=np.int32)
    tokens = np.array([70, 11, 12, 13, 14, 15, 16], dtype=np.int32)
    want_counts = np.array([1, 2], dtype=np.int32)
    want = np.array([0, 2, 5], dtype=np.int32)
    sizes = [7, 7, 7, 3, 2, 3, 2 * 3, 2 * 3]
    offsets = np.cumsum([0] + [(s + 3) // 4 * 4 for s in sizes[:-1]]).astype(np.int64)
    buf = np.full(int(offsets[-1]) + 8, -7, dtype=np.int32)
    starts, slots = np.empty(2, dtype=np.int32), np.empty(2, dtype=np.int32)
    row_request, row_version = np.full(2, -1, dtype=np.int64), np.full(2, -1, dtype=np.int64)

    def pack():
        code = m._lib.hbh_pack_step(m._ptr, 2, handles.ctypes.data, n_new.ctypes.data, tokens.ctypes.data,
                                    want_counts.ctypes.data, want.ctypes.data, np.array(widths, dtype=np.int32).ctypes.data,
                                    offsets.ctypes.data, buf.ctypes.data, starts.ctypes.data, slots.ctypes.data,
                                    row_request.ctypes.data, row_version.ctypes.data)
        assert code == 0

    pack()
    o = offsets
    assert buf[o[0]: o[0] + 7].tolist() == tokens.tolist()
    assert buf[o[1]: o[1] + 7].tolist() == [9, 0, 1, 2, 3, 4, 5]
    assert buf[o[2]: o[2] + 7].tolist() == [0, 1, 1, 1, 1, 1, 1]
    assert buf[o[3]: o[3] + 3].tolist() == [0, 1, 7]
    assert buf[o[4]: o[4] + 2].tolist() == [m.slot("a"), m.slot("b")] == slots.tolist()
    assert buf[o[5]: o[5] + 3].tolist() == [0, 1 + 2, 1 + 5] and starts.tolist() == [9, 0]
    for g in range(2):
        rows = buf[o[6 + g]: o[6 + g] + 6].reshape(2, 3)
        assert rows[0].tolist() == m.table(g, "a") and rows[1].tolist() == m.table(g, "b") + [-1]
    # nothing changed: the rows are left alone (a scribble survives); a row that held another
    # request, or an older state of the tables, is rewritten
    buf[o[6]] = 99
    pack()
    assert buf[o[6]] == 99
    row_request[0] = 12345
    pack()
    assert buf[o[6]] == m.table(0, "a")[0]
    buf[o[6]] = 99
    row_version[0] -= 1
    pack()
    assert buf[o[6]] == m.table(0, "a")[0] and row_version[0] == m.table_version("a")


def test_pool_sizes_from_a_byte_budget():
    """Without an explicit capacity the pools are sized from the memory that is free: windowed groups
    get what the live requests' windows need, the groups that keep every key the rest; nothing
    exceeds the budget, a cap on tokens holds, and a tiny budget still leaves every request pages."""
    from hi_b200.cache.device import bytes_per_token, pool_tokens_for_budget
    from hi_b200.parts.spec import CacheSpec

    keep, chunk = CacheSpec(8, 128, None), CacheSpec(8, 128, ("chunk", 8192))
    specs = {i: (keep if i % 4 == 3 else chunk) for i in range(16)}          # Scout: 4 global, 12 chunked layers
    cost = bytes_per_token(specs, 2)
    assert cost == [12 * 4096, 4 * 4096] or cost == [4 * 4096, 12 * 4096]
    from hi_b200.cache.device import plan_groups
    groups, _ = plan_groups(specs)
    g_keep = [g for g, s in enumerate(groups) if s.window is None][0]
    g_chunk = 1 - g_keep
    budget = 80 << 30
    tokens = pool_tokens_for_budget(specs, 2, budget, 64, 8)
    assert all(t % 64 == 0 for t in tokens)
    assert tokens[g_chunk] == 8 * (8192 + 128) + 8192
    used = sum(t * c for t, c in zip(tokens, cost))
    assert 0.99 * budget <= used <= budget
    capped = pool_tokens_for_budget(specs, 2, budget, 64, 8, most_tokens=100_000)
    assert capped[g_keep] == 100_032 and capped[g_chunk] == tokens[g_chunk]
    small = pool_tokens_for_budget(specs, 2, 1 << 20, 64, 8)
    assert all(t >= 2 * 64 for t in small)
    assert pool_tokens_for_budget({0: None}, 2, budget, 64, 8) == []

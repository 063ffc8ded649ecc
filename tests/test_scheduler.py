"""The scheduler's decisions, on the host: admission, token budget and portions, decoding,
finishing and freeing, and what happens when pages run out."""
import random

import pytest

from hi_b200.cache import CacheManager
from hi_b200.engine.scheduler import FINISHED, Request, Scheduler, SchedulerConfig
from hi_b200.parts.spec import CacheSpec
from hi_b200.sampling import SamplingParams

GLOBAL = CacheSpec(kv_heads=1, head_dim=16, window=None)
CHUNK = CacheSpec(kv_heads=1, head_dim=16, window=("chunk", 16))


def make(pages=(64, 64), page=4, slots=8, eos=(), max_len=None, **cfg):
    mgr = CacheManager([GLOBAL, CHUNK], list(pages), page_size=page, max_requests=slots)
    return mgr, Scheduler(mgr, SchedulerConfig(**cfg), eos_token_ids=eos, max_model_len=max_len)


def run_step(mgr, sched, next_token=lambda r: 1):
    """What the engine does with a plan: reserve and commit pages, 'sample', commit the plan."""
    plan = sched.plan()
    for e in plan.entries:
        rid = e.request.request_id
        if not mgr.is_open(rid):
            mgr.open(rid)
        mgr.reserve(rid, len(e.tokens))
    for e in plan.entries:
        mgr.commit(e.request.request_id, len(e.tokens))
    sampled = {e.request.request_id: next_token(e.request) for e in plan.entries if e.samples}
    done = sched.commit(plan, sampled)
    mgr.check_invariants()
    return plan, done


def req(rid, n, max_tokens=4, **kw):
    return Request(rid, list(range(1, n + 1)), SamplingParams(max_tokens=max_tokens, **kw))


def test_budget_cuts_prompts_into_portions_and_decodes_go_first():
    mgr, s = make(max_batched_tokens=10, max_batch_size=4)
    s.add(req("a", 23)); s.add(req("b", 5))
    p1, _ = run_step(mgr, s)
    assert [(e.request.request_id, len(e.tokens), e.samples) for e in p1.entries] == [("a", 10, False)]
    p2, _ = run_step(mgr, s)
    assert [(e.request.request_id, len(e.tokens)) for e in p2.entries] == [("a", 10)]
    p3, _ = run_step(mgr, s)       # a's last 3 tokens (sampled), b admitted into the rest of the budget
    assert [(e.request.request_id, len(e.tokens), e.samples) for e in p3.entries] == [("a", 3, True), ("b", 5, True)]
    p4, _ = run_step(mgr, s)       # both decode: one token each, in one batch
    assert [(e.request.request_id, e.tokens, e.samples) for e in p4.entries] == [("a", [1], True), ("b", [1], True)]
    assert p4.entries[0].request.computed == 24


def test_portions_respect_max_prefill_portion_and_batch_size():
    mgr, s = make(max_batched_tokens=100, max_batch_size=2, max_prefill_portion=7)
    for i in range(3):
        s.add(req(i, 20))
    p, _ = run_step(mgr, s)
    assert [(e.request.request_id, len(e.tokens)) for e in p.entries] == [(0, 7), (1, 7)]
    assert len(s.running) == 2 and len(s.waiting) == 1


def test_finish_on_length_and_on_eos_frees_everything():
    mgr, s = make(eos=(9,))
    s.add(req("a", 6, max_tokens=3)); s.add(req("b", 6, max_tokens=50)); s.add(req("c", 6, max_tokens=50, ignore_eos=True))
    toks = {"a": iter([5, 5, 5]), "b": iter([5, 9]), "c": iter([9, 9] + [5] * 60)}
    done = []
    while s.has_work():
        _, d = run_step(mgr, s, lambda r: next(toks[r.request_id]))
        done += d
    by = {r.request_id: r for r in done}
    assert by["a"].output == [5, 5, 5] and by["a"].finish_reason == "length"
    assert by["b"].output == [5] and by["b"].finish_reason == "stop"          # EOS is not emitted
    assert by["c"].output[:2] == [9, 9] and len(by["c"].output) == 50
    assert all(p.free == p.total for p in mgr.pools) and mgr.free_slots == 8 and not mgr.requests


def test_requests_are_validated_when_added():
    mgr, s = make(pages=(4, 4), page=4, max_len=64)
    with pytest.raises(ValueError, match="prompt is empty"):
        s.add(Request("e", [], SamplingParams()))
    with pytest.raises(ValueError, match="max_tokens"):
        s.add(req("m", 3, max_tokens=0))
    with pytest.raises(ValueError, match="temperature"):
        s.add(req("t", 3, temperature=-1.0))
    with pytest.raises(ValueError, match="top_p"):
        s.add(req("p", 3, top_p=1.5))
    with pytest.raises(ValueError, match="top_k"):
        s.add(req("k", 3, top_k=0))
    with pytest.raises(ValueError, match="context_length_exceeded"):
        s.add(req("l", 60, max_tokens=5))
    with pytest.raises(ValueError, match="insufficient_gpu_memory"):
        s.add(req("g", 14, max_tokens=4))          # 18 tokens need 5 pages of the global group; it has 4
    s.add(req("ok", 12, max_tokens=4))


def test_when_pages_run_out_prompts_shrink_and_wait_and_nothing_new_is_admitted():
    mgr, s = make(pages=(6, 6), page=4, max_batched_tokens=64, max_batch_size=4)
    s.add(req("a", 16, max_tokens=2)); s.add(req("b", 14, max_tokens=2))
    p1, _ = run_step(mgr, s)        # a takes 4 pages; b gets the 2 that are left: 8 of its 14 tokens
    assert [(e.request.request_id, len(e.tokens)) for e in p1.entries] == [("a", 16), ("b", 8)]
    assert s.counters["shrunk_portions"] == 1
    s.add(req("c", 4, max_tokens=2))
    p2, _ = run_step(mgr, s)        # a decodes (its 5th page would be needed: none free -> see below)
    ids = [e.request.request_id for e in p2.entries]
    assert "c" not in ids, "a new request was admitted while running ones lack pages"


def test_a_decode_that_cannot_get_a_page_preempts_the_youngest_request():
    mgr, s = make(pages=(6, 6), page=4, max_batched_tokens=64, max_batch_size=4)
    s.add(req("old", 11, max_tokens=8)); s.add(req("young", 11, max_tokens=8))
    run_step(mgr, s)                               # both prefilled: 3 + 3 pages, pool full
    plan, _ = run_step(mgr, s)                     # position 11 fits the third page of each
    assert len(plan.entries) == 2 and not plan.preempted
    plan, _ = run_step(mgr, s)                     # position 12 needs a 4th page: none -> young is preempted
    assert [r.request_id for r in plan.preempted] == ["young"]
    assert [e.request.request_id for e in plan.entries] == ["old"]
    young = plan.preempted[0]
    assert young.status == "waiting" and young.computed == 0 and young.preemptions == 1 and len(young.output) == 2
    assert s.waiting[0] is young and not mgr.is_open("young")
    # it comes back with prompt + generated tokens as its prompt once pages are free, and finishes
    while s.has_work():
        run_step(mgr, s)
    assert young.status == FINISHED and len(young.output) == 8 and young.finish_reason == "length"
    assert all(p.free == p.total for p in mgr.pools)


def test_two_prompts_that_fit_only_one_at_a_time_both_finish():
    """Two 96-token prompts, each of which fits the pool alone, cut into 16-token portions: the
    second is not admitted while the first is in its prompt (both would fill the pool and neither
    could go on); every request still finishes and nothing leaks."""
    mgr, s = make(pages=(32, 32), page=4, max_batched_tokens=64, max_batch_size=4, max_prefill_portion=16)
    a, b = req("a", 96, max_tokens=3), req("b", 96, max_tokens=3)
    s.add(a); s.add(b)
    p1, _ = run_step(mgr, s)
    assert [(e.request.request_id, len(e.tokens)) for e in p1.entries] == [("a", 16)]
    steps = 1
    while s.has_work():
        plan, _ = run_step(mgr, s)
        assert plan.entries or plan.preempted, "the scheduler stalled"
        steps += 1
        assert steps < 200
    assert a.status == FINISHED and b.status == FINISHED and len(a.output) == 3 and len(b.output) == 3
    assert all(p.free == p.total for p in mgr.pools) and not mgr.requests


def test_when_every_running_request_waits_for_a_page_the_youngest_is_preempted():
    """Both requests are in their prompts and hold the whole pool between them (pages taken by
    another user of the cache made the admission's estimate too kind): no step could run and no
    later step would free a page, so the youngest goes back to the queue and the older one moves."""
    mgr, s = make(pages=(32, 32), page=4, max_batched_tokens=64, max_batch_size=4, max_prefill_portion=16)
    a, b = req("a", 60, max_tokens=2), req("b", 60, max_tokens=2)
    s.add(a); s.add(b)
    run_step(mgr, s)                                   # a 16, and b 16: both fit to the end (15 + 15 pages)
    assert [r.request_id for r in s.running] == ["a", "b"]
    mgr.open("guest"); mgr.reserve("guest", 4 * 24)     # someone else takes 24 pages of each group
    plan, _ = run_step(mgr, s)                         # nothing is free: b is preempted, a moves on
    assert [r.request_id for r in plan.preempted] == ["b"] and b.preemptions == 1
    assert [(e.request.request_id, len(e.tokens)) for e in plan.entries] == [("a", 16)]
    mgr.close("guest")
    while s.has_work():
        plan, _ = run_step(mgr, s)
        assert plan.entries or plan.preempted
    assert a.status == FINISHED and b.status == FINISHED and len(b.output) == 2
    assert all(p.free == p.total for p in mgr.pools) and not mgr.requests


def test_seeded_generators_survive_preemption():
    r = req("x", 3, temperature=1.0, seed=42)
    first = [r.rng.next_f32() for _ in range(3)]
    r2 = req("y", 3, temperature=1.0, seed=42)
    assert [r2.rng.next_f32() for _ in range(3)] == first and all(0.0 <= u < 1.0 for u in first)


@pytest.mark.parametrize("seed", range(4))
def test_random_workloads_finish_and_leak_nothing(seed):
    rng = random.Random(seed)
    mgr, s = make(pages=(rng.randint(12, 24),) * 2, page=4, slots=4, max_batched_tokens=rng.choice([8, 16, 40]),
                  max_batch_size=3, max_active_requests=4, max_prefill_portion=rng.choice([None, 5]))
    reqs = [req(i, rng.randint(1, 30), max_tokens=rng.randint(1, 12)) for i in range(12)]
    pending = list(reqs)
    steps = 0
    while pending or s.has_work():
        if pending and rng.random() < 0.5:
            s.add(pending.pop(0))
        if s.has_work():
            plan, _ = run_step(mgr, s, lambda r: rng.randrange(3, 50))
            assert plan.n_tokens <= s.config.max_batched_tokens and len(plan.entries) <= 3
            assert plan.entries or plan.preempted
        steps += 1
        assert steps < 5000, "the scheduler does not make progress"
    assert all(r.status == FINISHED and len(r.output) == r.params.max_tokens for r in reqs)
    assert all(p.free == p.total for p in mgr.pools) and mgr.free_slots == 4


def run_ahead(mgr, sched, token_of):
    """The loop of a caller that plans step t+1 while step t still runs: the plan is 'launched'
    (pages reserved and committed) at once, the step before it is committed only afterwards."""
    in_flight, done, steps = None, [], 0
    while sched.has_work() or in_flight is not None:
        plan = sched.plan() if sched.has_work() else None
        if plan is not None:
            for e in plan.entries:
                rid = e.request.request_id
                if not mgr.is_open(rid):
                    mgr.open(rid)
                mgr.reserve(rid, len(e.tokens))
            for e in plan.entries:
                mgr.commit(e.request.request_id, len(e.tokens))
        if in_flight is not None:
            sampled = {e.request.request_id: token_of(e.request) for e in in_flight.entries if e.samples}
            done += sched.commit(in_flight, sampled)
        mgr.check_invariants()
        in_flight = plan if plan is not None and plan.entries else None
        steps += 1
        assert steps < 5000, "the scheduler does not make progress"
    return done


@pytest.mark.parametrize("seed", range(4))
def test_planning_one_step_ahead_gives_the_same_outputs(seed):
    """Planning step t+1 before step t is committed: the entries of t+1 hold IN_FLIGHT where t's
    sample goes, a request that stops at t leaves a void entry in t+1, preemption still works, and
    every request ends with the tokens and the reason it has when each step is committed at once."""
    from hi_b200.engine.scheduler import IN_FLIGHT

    def token_of(r):             # the next token is a function of the request and how far it is
        return 9 if (r.request_id * 7 + len(r.output)) % 11 == 5 else 20 + (r.request_id + len(r.output)) % 30

    def workload():
        rng = random.Random(seed)
        return [req(i, rng.randint(1, 30), max_tokens=rng.randint(1, 14)) for i in range(10)]

    results = []
    for ahead in (False, True):
        rng = random.Random(100 + seed)
        mgr, s = make(pages=(rng.randint(10, 20),) * 2, page=4, slots=4, eos=(9,), max_batched_tokens=rng.choice([8, 24]),
                      max_batch_size=3, max_active_requests=4)
        for r in workload():
            s.add(r)
        if ahead:
            done = run_ahead(mgr, s, token_of)
        else:
            done = []
            while s.has_work():
                done += run_step(mgr, s, token_of)[1]
        assert len(done) == 10 and all(p.free == p.total for p in mgr.pools) and mgr.free_slots == 4 and not mgr.requests
        results.append({r.request_id: (r.output, r.finish_reason) for r in done})
        assert all(9 not in out for out, _ in results[-1].values()), "the end-of-sequence token was emitted"
    assert results[0] == results[1]
    assert {reason for _, reason in results[0].values()} == {"stop", "length"}


def test_a_plan_made_ahead_marks_the_token_in_flight_and_a_third_plan_is_refused():
    from hi_b200.engine.scheduler import IN_FLIGHT

    mgr, s = make()
    s.add(req("a", 5, max_tokens=3))
    p1 = s.plan()
    assert [(e.tokens, e.samples) for e in p1.entries] == [([1, 2, 3, 4, 5], True)]
    p2 = s.plan()                                     # before p1 is committed: a's next token is not known yet
    assert [(e.tokens, e.samples) for e in p2.entries] == [([IN_FLIGHT], True)]
    with pytest.raises(RuntimeError, match="outstanding"):
        s.plan()
    assert s.commit(p1, {"a": 40}) == [] and p2.entries[0].request.output == [40]
    p3 = s.plan()                                     # the third and last token: still ahead of p2's commit
    assert [(e.tokens, e.samples) for e in p3.entries] == [([IN_FLIGHT], True)]
    assert s.commit(p2, {"a": 41}) == []
    p4 = s.plan()                                     # nothing left to plan: a waits for its last sample
    assert p4.entries == [] and s.commit(p4, {}) == []
    with pytest.raises(RuntimeError, match="order"):
        s.commit(p2, {"a": 41})                       # p2 is committed already
    done = s.commit(p3, {"a": 42})
    assert [r.request_id for r in done] == ["a"] and done[0].output == [40, 41, 42] and done[0].finish_reason == "length"
    assert not s.has_work()


def test_abort_of_waiting_running_and_in_flight_requests():
    """abort() between steps: a waiting request never runs; a running one gives its pages and its
    slot back at once; one that has an entry in a plan made ahead leaves that entry void (it runs,
    nobody reads it); an unknown id is refused. The others go on to their ends."""
    mgr, s = make(pages=(64, 64), page=4, slots=3, max_batched_tokens=64, max_batch_size=3, max_active_requests=3)
    reqs = {n: req(n, 9, max_tokens=6) for n in "abcd"}
    for r in reqs.values():
        s.add(r)
    run_step(mgr, s)                                   # a, b, c are prefilled; d waits for a slot
    assert [r.request_id for r in s.waiting] == ["d"]
    assert s.abort("d") is reqs["d"] and reqs["d"].finish_reason == "aborted" and not s.waiting
    assert s.abort("nobody") is None and s.abort("d") is None
    used = mgr.pools[0].total - mgr.pools[0].free
    assert s.abort("b") is reqs["b"] and not mgr.is_open("b")
    assert mgr.pools[0].total - mgr.pools[0].free == used - 3 and mgr.free_slots == 1
    mgr.check_invariants()
    # a plan made ahead holds an entry of c; c is aborted before that plan is committed
    p1 = s.plan()
    for e in p1.entries:
        mgr.reserve(e.request.request_id, len(e.tokens)); mgr.commit(e.request.request_id, len(e.tokens))
    p2 = s.plan()
    assert sorted(e.request.request_id for e in p2.entries) == ["a", "c"]
    assert s.abort("c") is reqs["c"] and not mgr.is_open("c")
    before = len(reqs["c"].output)
    s.commit(p1, {"a": 5, "c": 5})
    for e in p2.entries:
        if mgr.is_open(e.request.request_id):
            mgr.reserve(e.request.request_id, len(e.tokens)); mgr.commit(e.request.request_id, len(e.tokens))
    s.commit(p2, {"a": 6, "c": 6})
    assert len(reqs["c"].output) == before and reqs["c"].status == FINISHED
    while s.has_work():
        run_step(mgr, s)
    assert reqs["a"].finish_reason == "length" and len(reqs["a"].output) == 6
    assert all(p.free == p.total for p in mgr.pools) and mgr.free_slots == 3 and not mgr.requests

"""Captured decode steps (CUDA graphs) against the plain model: the path that generation and the
benchmark take. A step of single tokens that all want their logits is captured once per (batch
size, context bucket) and replayed from static buffers; block-table rows are rewritten only
when another request sits in them or the request's tables changed. These tests cross bucket
edges, let rows change owner, free windowed pages under a captured step (entries of -1 at the
head of a table), evict graphs and capture them again, and make a step report a failed wait."""
import pytest
import torch

import harness as h
from tiny_configs import TINY_A, TINY_D

pytestmark = pytest.mark.gpu

DTYPES = [("float32", h.TOL_F32), ("bfloat16", h.TOL_BF16)]

# head_dim 64, chunks of 64 positions and 16-token pages: the shapes at which the tensor-core decode
# kernel loads its tiles by TMA, with a chunk edge every 64 tokens
TINY_D64 = dict(TINY_D, attention_chunk_size=64)


def decode_trace(reqs, prefill, order_after=None, leave=None, join=None):
    """Prompts whole (logits at their last token), then every live request decodes one token per
    step in one batch. ``leave = (rid, step)``: the request ends after that many decode steps;
    ``join = (rid, step)``: a request whose prompt is fed at that step and which decodes from then
    on, placed FIRST in the batch so that every row changes owner."""
    steps = []
    done = {}
    live = []
    for rid, toks in reqs.items():
        if join and rid == join[0]:
            continue
        n = prefill[rid]
        steps.append(([(rid, toks[:n], [n - 1])], []))
        done[rid] = n
        live.append(rid)
    t = 0
    while live:
        if join and t == join[1]:
            rid = join[0]
            n = prefill[rid]
            steps.append(([(rid, reqs[rid][:n], [n - 1])], []))
            done[rid] = n
            live.insert(0, rid)
        entries, end = [], []
        for rid in list(live):
            entries.append((rid, [reqs[rid][done[rid]]], [0]))
            done[rid] += 1
            if done[rid] == len(reqs[rid]) or (leave and rid == leave[0] and t + 1 == leave[1]):
                end.append(rid)
                live.remove(rid)
        steps.append((entries, end))
        t += 1
    return steps


def run_and_compare(cfg, mdir, dtype, tol, steps, reqs, what, **engine_options):
    from hi_b200.engine.core import Engine

    eng = Engine.from_dir(mdir, dtype=dtype, **engine_options)
    got, forced = h.replay_in_process(eng, steps, record_routing=(dtype == "bfloat16"))
    # only the positions that were fed count (a request that leaves early is cut short)
    fed = {}
    for entries, _ in steps:
        for rid, toks, _w in entries:
            fed[rid] = fed.get(rid, 0) + len(toks)
    cut = {rid: toks[:fed[rid]] for rid, toks in reqs.items()}
    h.compare_with_plain(cfg, h.read_weights(mdir), cut, got, tol, forced=forced if dtype == "bfloat16" else None,
                         what=what, margin=h.ROUTING_MARGIN)
    assert not eng.manager.requests
    for pool in eng.manager.pools:
        assert pool.free == pool.total, "pages were lost"
    return eng


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("name", ["A", "D"])
def test_decoding_across_a_context_bucket_with_rows_that_change_owner(name, dtype, tol, model_dirs):
    """Two requests decode from about 1,000 cached tokens across position 1,024 (the default
    bucket: the step is captured again with wider tables), a short one beside them ends in the
    middle, and a fourth joins at the head of the batch, so each table row gets another request."""
    cfg, mdir = model_dirs[name + "_small_std"]
    lengths = {"long": 1062, "near": 1050, "short": 60, "late": 75}
    reqs = {rid: h.random_tokens(cfg, n, seed=300 + i) for i, (rid, n) in enumerate(lengths.items())}
    prefill = {"long": 1002, "near": 1013, "short": 30, "late": 40}
    steps = decode_trace(reqs, prefill, leave=("short", 17), join=("late", 25))
    assert max(len(e) for e, _ in steps) == 3
    eng = run_and_compare(cfg, mdir, dtype, tol, steps, reqs, f"bucket edge {name} {dtype}", kv_page_size=16,
                          kv_cache_tokens=2400, max_active_requests=4)
    buckets = sorted({bucket for (_n, bucket) in eng._graphs})
    assert buckets == [1024, 2048], f"decode steps were captured for buckets {buckets}"
    assert all(g.captured for g in eng._graphs.values())


@pytest.mark.parametrize("dtype,tol", DTYPES)
def test_freed_chunks_under_captured_steps_and_graphs_that_are_evicted(dtype, tol, tmp_path):
    """Three requests decode 200 tokens each, token by token, over three chunk edges, with
    16-token pages, buckets of 32 tokens and room for three graphs: windowed pages are freed under
    captured steps (their table entries turn -1), tables grow past the captured width every other
    page, graphs are evicted and captured again; in bfloat16 the keys come in by TMA."""
    from hi_b200.kernels import ops

    cfg = TINY_D64
    mdir = h.make_model(str(tmp_path / "m"), cfg, seed=21, std=0.02)
    lengths = {"a": 215, "b": 190, "c": 140}
    reqs = {rid: h.random_tokens(cfg, n, seed=400 + i) for i, (rid, n) in enumerate(lengths.items())}
    prefill = {"a": 15, "b": 3, "c": 70}
    steps = decode_trace(reqs, prefill)
    before = dict(ops.CALLS)
    eng = run_and_compare(cfg, mdir, dtype, tol, steps, reqs, f"freed chunks under graphs {dtype}", kv_page_size=16,
                          kv_cache_tokens=720, windowed_cache_tokens=288, max_active_requests=3,
                          graph_context_bucket=32, max_graphs=3, debug_poison=True)
    assert len(eng._graphs) <= 3
    chunked = [g for g in eng.manager.snapshot()["groups"] if g["window"]]
    assert chunked and chunked[0]["peak"] <= 3 * (64 // 16 + 1), "the chunked group kept pages of dead chunks"
    assert chunked[0]["allocations"] > chunked[0]["total"], "pages of dead chunks were not used again"
    if dtype == "bfloat16":
        assert ops.CALLS.get("attention_decode_fused", 0) > before.get("attention_decode_fused", 0), \
            "the fused TMA decode kernel did not run"


def test_a_captured_step_equals_the_same_step_run_eagerly(model_dirs):
    """The same decode steps with and without graphs give the same logits, bit for bit: a graph
    holds the eager step's own kernels (its attention splits are cut for the bucket's width, the
    eager step's for the longest context, which moves sums by rounding only in bfloat16; float32
    attention adds in one fixed order per token)."""
    from hi_b200.engine.core import Engine

    cfg, mdir = model_dirs["A"]
    reqs = {rid: h.random_tokens(cfg, n, seed=500 + i) for i, (rid, n) in enumerate((("x", 90), ("y", 70)))}
    steps = decode_trace(reqs, {"x": 20, "y": 9})
    runs = []
    for graphs in (True, False):
        eng = Engine.from_dir(mdir, dtype="float32", kv_page_size=8, kv_cache_tokens=256, max_active_requests=2,
                              use_cuda_graphs=graphs, graph_context_bucket=64)
        got, _ = h.replay_in_process(eng, steps)
        runs.append(got)
        assert bool(eng._graphs) == graphs
    for rid in reqs:
        for p, row in runs[0][rid].items():
            assert (row == runs[1][rid][p]).all(), f"request {rid} position {p}: the captured step differs"


def test_a_failed_wait_in_a_step_launched_ahead_aborts_instead_of_committing(tmp_path):
    """Kernels with bounded waits leave a code in a status word when a wait runs out. Here the
    word is set from the host (nothing on the GPU fails): the entry point must raise before it
    commits that step's tokens, abort the requests of that step and of the one launched on top of
    it, and leave the cache whole."""
    import hi_b200
    from hi_b200.kernels import ops

    cfg = dict(TINY_D64)
    mdir = h.make_model(str(tmp_path / "m"), cfg, seed=5, std=0.02)
    llm = hi_b200.LLM(mdir, dtype="bfloat16", kv_page_size=16, kv_cache_tokens=512, max_batch_size=2)
    reqs = [llm.add_request(h.random_tokens(cfg, n, seed=n), hi_b200.SamplingParams(max_tokens=40, ignore_eos=True))
            for n in (20, 33)]
    for _ in range(8):
        llm.step()
    assert llm.engine._graphs and all(len(r.output) >= 4 for r in reqs)
    assert llm._launched is not None and llm._launched.status is not None, "decode steps should carry a status ticket"
    torch.cuda.synchronize()
    committed = [len(r.output) for r in reqs]
    ops._tc_status(llm.engine.device).fill_(31)          # as if the next step's attention had given up a wait
    llm.step()                                           # launches a step (its ticket carries the code) and reads the one before
    with pytest.raises(ops.KernelError, match="bounded wait"):
        for _ in range(3):
            llm.step()
    assert all(r.status == "finished" and r.finish_reason == "aborted" for r in reqs)
    assert [len(r.output) for r in reqs] <= [c + 1 for c in committed], "tokens of the failed step were committed"
    llm.engine.manager.check_invariants()
    assert not llm.engine.manager.requests and all(p.free == p.total for p in llm.engine.manager.pools)
    # the engine goes on: the word was cleared when it was read
    out = llm.generate([h.random_tokens(cfg, 12, seed=1)], hi_b200.SamplingParams(max_tokens=5, ignore_eos=True))
    assert out[0].completion_tokens == 5


def test_an_earlier_engine_that_becomes_garbage_while_a_step_is_captured(model_dirs):
    """An engine and its captured steps refer to each other, so Python frees them whenever its
    cycle collector happens to run; freeing a CUDA graph is not allowed while a stream is being
    captured. Here the old engine becomes garbage in the middle of the new engine's capture, and
    enough objects are made there for the collector to run: the capture must come through."""
    import gc

    from hi_b200.engine.core import Engine, StepEntry

    cfg, mdir = model_dirs["A"]
    toks = h.random_tokens(cfg, 40, seed=77)

    def started():
        eng = Engine.from_dir(mdir, dtype="float32", kv_page_size=8, kv_cache_tokens=128, max_active_requests=1)
        eng.step([StepEntry("a", toks[:20], [19])])
        return eng

    gc.collect()
    was_enabled, thresholds, watch = gc.isenabled(), gc.get_threshold(), None
    gc.disable()                               # every object made from here on stays in the youngest generation
    try:
        old = started()
        for p in range(20, 24):                # one eager step, the capture, two replays
            old.step([StepEntry("a", [toks[p]], [0])])
        assert old._graphs
        holder = [old]
        del old
        new = started()
        new.step([StepEntry("a", [toks[20]], [0])])              # the shape's first step runs eagerly
        inner = new.model.forward

        def forward(*args):
            if torch.cuda.is_current_stream_capturing() and holder:
                holder.clear()                                    # the old engine is garbage from here on
                _churn = [[i] for i in range(200000)]             # container objects: the collector's trigger
            return inner(*args)

        new.model.forward = forward
        during = []                            # collections that started while the stream was being captured
        watch = lambda phase, info: during.append(info["generation"]) \
            if phase == "start" and torch.cuda.is_current_stream_capturing() else None
        gc.callbacks.append(watch)
        gc.set_threshold(gc.get_count()[0] + 50000, 1, 1)        # no collection before the capture: the old engine
        gc.enable()                                               # stays in the youngest generation till then
        got = new.step([StepEntry("a", [toks[21]], [0])])         # captured here
        assert not during, "the cycle collector ran inside the capture"
        assert not holder and new._graphs and torch.isfinite(got).all()
        again = new.step([StepEntry("a", [toks[22]], [0])])
        assert torch.isfinite(again).all()
    finally:
        if watch in gc.callbacks:
            gc.callbacks.remove(watch)
        gc.set_threshold(*thresholds)
        (gc.enable if was_enabled else gc.disable)()
    new.finish("a")

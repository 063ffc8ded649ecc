"""bin/trace_run, run as a user would, against the plain model: each request alone and whole;
most of it in one step and the last 32 tokens one by one; portions of changing size; and
mixed batches with so few pages that they are used again. float32 and bfloat16."""
import pytest

import harness as h

pytestmark = pytest.mark.gpu

# request lengths: BASELINE's workloads (prompt + decoded tokens) plus longer ones that cross
# several 64-token pages and attention chunks, so pages of dead chunks and of finished
# requests come round again
LENGTHS = {"A": [7 + 16, 19 + 16, 33 + 16, 48 + 16, 150, 201], "B": [5 + 24, 40 + 24, 70 + 24, 131, 190]}


def build(cfg, name):
    reqs = {f"r{i}": h.random_tokens(cfg, n, seed=100 + i) for i, n in enumerate(LENGTHS[name])}
    traces = {
        "whole": h.trace_whole(reqs),
        "tail": h.trace_tail_decode(reqs),
        "portions": h.trace_portions(reqs),
        "mixed": h.trace_mixed(reqs, max_tokens=576, page=64, seed=3),
    }
    steps, owners = [], {}
    for regime, tr in traces.items():
        for entries, end in tr:
            steps.append(([(f"{regime}:{r}", t, w) for r, t, w in entries], [f"{regime}:{r}" for r in end]))
    all_reqs = {f"{regime}:{r}": toks for regime in traces for r, toks in reqs.items()}
    return steps, all_reqs


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_regimes(name, dtype, model_dirs, tmp_path):
    cfg, mdir = model_dirs[name]
    weights = h.read_weights(mdir)
    steps, reqs = build(cfg, name)
    live_peak = max(len(e) for e, _ in steps)
    assert live_peak >= 3, "the mixed regime must hold several requests at once"
    if dtype == "float32":
        got = h.replay_subprocess(mdir, dtype, steps, 576, str(tmp_path / "out"), h.vocab_of(cfg))
        h.compare_with_plain(cfg, weights, reqs, got, h.TOL_F32, what=f"{name} {dtype}")
    else:
        got, forced = h.replay_subprocess(mdir, dtype, steps, 576, str(tmp_path / "out"), h.vocab_of(cfg),
                                          dump_taps=True)
        h.compare_with_plain(cfg, weights, reqs, got, h.TOL_BF16, forced=forced, what=f"{name} {dtype}",
                             margin=h.ROUTING_MARGIN)
    for rid, toks in reqs.items():
        assert sorted(got[rid]) == list(range(len(toks))), f"{rid}: not every position came back"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_with_small_pages_and_a_chunk_pool_of_its_own(dtype, model_dirs, tmp_path):
    """--page-size 8 with --num-pages-chunk 5: tiny A's chunked layer (32 positions = 4 pages) lives
    in five pages while the global layer has room for the whole request; the mixed regime then
    needs the pages of dead chunks at once."""
    cfg, mdir = model_dirs["A"]
    weights = h.read_weights(mdir)
    reqs = {"a": h.random_tokens(cfg, 150, seed=31)}
    steps = h.trace_portions(reqs, sizes=(7, 2, 1, 5, 8, 3, 1, 1, 6))
    kw = dict(extra=["--page-size", "8", "--num-pages-global", "19", "--num-pages-chunk", "5", "--max-live", "1"])
    if dtype == "float32":
        got = h.replay_subprocess(mdir, dtype, steps, 152, str(tmp_path / "out"), h.vocab_of(cfg), **kw)
        h.compare_with_plain(cfg, weights, reqs, got, h.TOL_F32, what=f"small pages {dtype}")
    else:
        got, forced = h.replay_subprocess(mdir, dtype, steps, 152, str(tmp_path / "out"), h.vocab_of(cfg), dump_taps=True, **kw)
        h.compare_with_plain(cfg, weights, reqs, got, h.TOL_BF16, forced=forced, what=f"small pages {dtype}",
                             margin=h.ROUTING_MARGIN)
    # a portion that would need a sixth page of the chunk pool is refused, in words
    import subprocess, sys, os
    trace = h.trace_json([([("a", reqs["a"][:60], [])], [])])
    proc = subprocess.run([sys.executable, os.path.join(h.ROOT, "bin", "trace_run"), "--model", mdir, "--dtype", dtype,
                           "--out", str(tmp_path / "o2"), "--max-tokens", "152", "--page-size", "8", "--num-pages-chunk", "5"],
                          input=trace, capture_output=True, text=True, timeout=600)
    assert proc.returncode != 0 and "insufficient_gpu_memory" in proc.stderr

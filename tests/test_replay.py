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
                             margin=0.1)
    for rid, toks in reqs.items():
        assert sorted(got[rid]) == list(range(len(toks))), f"{rid}: not every position came back"

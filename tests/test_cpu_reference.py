"""The CPU reference (plain C++ loops in the host runtime, ``hi_b200/engine/cpu_reference.py``)
against the test-suite's plain model: two statements of the formulas, written apart, that must
agree on whole sequences of the four tiny configurations, with forced expert choices, with a
schedule that names a layer twice, in greedy and in seeded sampled generation, and through
``python -m hi_b200 run --cpu``. No GPU."""
import dataclasses
import json

import numpy as np
import pytest
import torch

import harness as h
import plain_llama4 as plain
from test_cli import run_cli

TOL = 1e-5     # relative to the largest |logit|: the two add in different orders, both in float32


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_the_two_plain_implementations_agree(name, model_dirs):
    from hi_b200.engine.cpu_reference import CpuReference

    cfg, mdir = model_dirs[name]
    w = h.read_weights(mdir)
    ref = CpuReference.from_dir(mdir)
    for n, seed in ((1, 0), (37, 1), (120, 2)):
        toks = h.random_tokens(cfg, n, seed=seed)
        records = {}
        want = plain.forward(cfg, w, toks, record=lambda nm, ids, gap: records.__setitem__(nm, (ids, gap)))
        got, routing = ref.forward(toks, return_routing=True)
        assert h.rel_err(got, want) <= TOL, f"{name}, {n} tokens"
        for nm, (ids, gap) in records.items():
            differs = (ids.sort(-1).values != routing[nm].long().sort(-1).values).any(-1)
            assert not bool((differs & (gap > 1e-4)).any()), f"{name} {nm}: expert choices differ"
        rows = [0, n - 1]
        assert torch.equal(ref.forward(toks, want=rows), got[rows])


def test_forced_choices_and_a_layer_named_twice(model_dirs):
    from hi_b200.config.registry import load_architecture
    from hi_b200.engine.cpu_reference import CpuReference
    from hi_b200.parts.model import Model
    from hi_b200.parts.spec import ScheduleEntry
    from hi_b200.weights.loader import load_from_dir

    cfg, mdir = model_dirs["B"]
    w = h.read_weights(mdir)
    toks = h.random_tokens(cfg, 50, seed=5)
    ref = CpuReference.from_dir(mdir)
    g = torch.Generator().manual_seed(3)
    forced = {f"model.layers.{i}.feed_forward": torch.stack([torch.randperm(8, generator=g)[:2] for _ in toks])
              for i in (1, 3, 5)}
    want = plain.forward(cfg, w, toks, forced_routing=forced)
    got, taken = ref.forward(toks, forced_routing=forced, return_routing=True)
    assert h.rel_err(got, want) <= TOL
    assert all(torch.equal(taken[n].long(), forced[n]) for n in forced)
    with pytest.raises(ValueError, match="refused"):
        ref.forward(toks, forced_routing={"model.layers.1.feed_forward": torch.full((50, 2), 8)})
    with pytest.raises(ValueError, match="refused"):
        ref.forward([0, 515])
    # the order of layers is data here too
    cfg_a, mdir_a = model_dirs["A"]
    arch, typed, _ = load_architecture(mdir_a)
    order = [0, 1, 0, 1, 1]
    spec = dataclasses.replace(arch.build_spec(typed), schedule=tuple(ScheduleEntry(layer=l, cache=i) for i, l in enumerate(order)))
    model = Model(spec, torch.float32, "cpu")
    load_from_dir(model, mdir_a, arch.normalize_tensor_name, arch.derive_tensors)
    toks = h.random_tokens(cfg_a, 40, seed=6)
    assert h.rel_err(CpuReference(model).forward(toks), plain.forward(cfg_a, h.read_weights(mdir_a), toks, schedule=order)) <= TOL


def test_generation_on_the_cpu_and_the_command_line(model_dirs):
    from hi_b200.engine.cpu_reference import CpuReference
    from hi_b200.sampling import SamplingParams

    cfg, mdir = model_dirs["A"]
    w = h.read_weights(mdir)
    prompt = h.random_tokens(cfg, 12, seed=9)
    ref = CpuReference.from_dir(mdir)
    out = ref.generate(prompt, 6)
    seq = list(prompt)
    for tok in out:
        assert tok == int(plain.forward(cfg, w, seq)[-1].argmax())
        seq.append(tok)
    # sampled: the plain sampler with the same generator gives the same tokens
    sp = SamplingParams(max_tokens=6, temperature=0.9, seed=4, ignore_eos=True)
    sampled = ref.generate(prompt, 6, sp)
    rng, seq = plain.Lcg(4), list(prompt)
    for tok in sampled:
        assert tok == plain.sample(plain.forward(cfg, w, seq)[-1], 0.9, 1.0, 0, rng.next_f32())
        seq.append(tok)
    res = run_cli("run", mdir, "--cpu", "--tokens", ",".join(map(str, prompt)), "--max-tokens", "6", "--top-k", "3",
                  "--dtype", "float32", "--include-logits")
    assert res.returncode == 0, res.stderr[-2000:]
    js = json.loads(res.stdout)
    assert js["backend"] == "hi_b200-cpu-reference-float32" and js["generated_tokens"] == out
    last = plain.forward(cfg, w, prompt)[-1]
    assert js["next_token"] == int(last.argmax()) == js["top_logits"][0]["token_id"] and js["logit_count"] == 256
    assert np.allclose(js["logits"], last.numpy(), atol=1e-4)


def test_text_in_and_out_where_the_folder_has_a_tokenizer(model_dirs, tmp_path):
    """--prompt and the text fields of `run`: with a tokenizer.json in the model folder (a word-level
    one made here) the prompt is encoded without special tokens and the outputs are decoded; without
    one --prompt is refused and the text fields stay empty."""
    import shutil

    tokenizers = pytest.importorskip("tokenizers")
    cfg, mdir = model_dirs["A"]
    d = str(tmp_path / "with_tokenizer")
    shutil.copytree(mdir, d)
    vocab = {f"w{i}": i for i in range(256)}
    tok = tokenizers.Tokenizer(tokenizers.models.WordLevel(vocab, unk_token="w0"))
    tok.pre_tokenizer = tokenizers.pre_tokenizers.Whitespace()
    tok.decoder = tokenizers.decoders.WordPiece(prefix="##")
    tok.save(d + "/tokenizer.json")
    res = run_cli("run", d, "--cpu", "--prompt", "w5 w17 w3 w200", "--max-tokens", "3", "--top-k", "2", "--dtype", "float32")
    assert res.returncode == 0, res.stderr[-2000:]
    js = json.loads(res.stdout)
    assert js["input_tokens"] == [5, 17, 3, 200]
    assert js["next_text"] == f"w{js['next_token']}" and js["top_logits"][0]["token"] == f"w{js['top_logits'][0]['token_id']}"
    assert js["generated_text"].split() == [f"w{t}" for t in js["generated_tokens"]]
    bare = run_cli("run", mdir, "--cpu", "--prompt", "w5", "--dtype", "float32")
    assert bare.returncode != 0 and "tokenizer.json" in bare.stderr


@pytest.mark.parametrize("name", ["A", "B"])
def test_trace_run_on_the_cpu_in_the_four_ways_of_cutting(name, model_dirs, tmp_path):
    """bin/trace_run --cpu, run as a user would where there is no GPU: the CPU arm of the replay.
    Whole, the last 32 tokens one by one, portions down to two tokens, and mixed with other
    requests; every row against the test-suite's plain model."""
    cfg, mdir = model_dirs[name]
    lengths = {"A": [23, 49, 64, 150], "B": [29, 94, 131]}[name]
    reqs = {f"r{i}": h.random_tokens(cfg, n, seed=300 + i) for i, n in enumerate(lengths)}
    traces = {"whole": h.trace_whole(reqs), "tail": h.trace_tail_decode(reqs), "portions": h.trace_portions(reqs),
              "mixed": h.trace_mixed(reqs, max_tokens=448, page=64, seed=5)}
    steps = [([(f"{regime}:{r}", t, w) for r, t, w in entries], [f"{regime}:{r}" for r in end])
             for regime, tr in traces.items() for entries, end in tr]
    all_reqs = {f"{regime}:{r}": toks for regime in traces for r, toks in reqs.items()}
    got = h.replay_subprocess(mdir, "float32", steps, 448, str(tmp_path / "out"), h.vocab_of(cfg), extra=["--cpu"])
    h.compare_with_plain(cfg, h.read_weights(mdir), all_reqs, got, TOL, what=f"trace_run --cpu, tiny {name}")
    for rid, toks in all_reqs.items():
        assert sorted(got[rid]) == list(range(len(toks))), f"{rid}: not every position came back"


def test_trace_run_on_the_cpu_refuses_what_it_cannot_mean(model_dirs, tmp_path):
    import os
    import subprocess
    import sys

    _cfg, mdir = model_dirs["A"]
    base = [sys.executable, os.path.join(h.ROOT, "bin", "trace_run"), "--model", mdir, "--out", str(tmp_path / "o"),
            "--max-tokens", "64", "--cpu"]
    proc = subprocess.run(base + ["--dtype", "bfloat16"], input="", capture_output=True, text=True, timeout=300)
    assert proc.returncode != 0 and "float32" in proc.stderr
    trace = h.trace_json([([("a", [1, 2, 3], [3])], [])])
    proc = subprocess.run(base + ["--dtype", "float32"], input=trace, capture_output=True, text=True, timeout=300)
    assert proc.returncode != 0 and "outside its tokens" in proc.stderr

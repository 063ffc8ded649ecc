"""The command line: `inspect` (CPU) and `run` (GPU), JSON in the shape of the reference's
`hi-local qwen-cpu` output (crates/hi-cuda/src/qwen_cpu.rs:62-81)."""
import json
import os
import subprocess
import sys

import pytest

import harness as h
import plain_llama4 as plain
from tiny_configs import TINY_A, TINY_B

ROOT = h.ROOT


def run_cli(*args):
    env = dict(os.environ, PYTHONPATH=ROOT)
    return subprocess.run([sys.executable, "-m", "hi_b200", *args], capture_output=True, text=True, env=env, timeout=600)


def test_inspect_and_random_weights(tmp_path):
    cfg = tmp_path / "c.json"
    cfg.write_text(json.dumps(TINY_B))
    out = run_cli("random-weights", str(cfg), str(tmp_path / "m"), "--seed", "3")
    assert out.returncode == 0, out.stderr
    rep = run_cli("inspect", str(tmp_path / "m"))
    assert rep.returncode == 0, rep.stderr
    info = json.loads(rep.stdout)
    assert info["tensors"]["status"] == "ok" and info["architecture"] == "llama4_text"
    assert [l["feed_forward"] for l in info["layers"]] == ["dense_swiglu", "moe_sigmoid"] * 3
    assert info["layers"][3]["window"] is None and info["layers"][0]["window"] == ["chunk", 16]
    os.remove(tmp_path / "m" / "model.safetensors")
    bad = run_cli("inspect", str(tmp_path / "m"))
    assert bad.returncode != 0 or json.loads(bad.stdout)["tensors"]["status"] == "error"


def test_token_list_parser():
    from hi_b200.cli import parse_token_ids

    assert parse_token_ids("1,2, 3\n4") == [1, 2, 3, 4]
    with pytest.raises(ValueError):
        parse_token_ids("1,x")


def test_engine_refuses_a_cpu_device(tmp_path):
    from hi_b200.engine.core import Engine

    d = h.make_model(str(tmp_path / "m"), TINY_A, seed=1)
    with pytest.raises(RuntimeError, match="CUDA"):
        Engine.from_dir(d, dtype="float32", device="cpu")


@pytest.mark.gpu
def test_run_prints_the_reference_shaped_json(tmp_path):
    d = h.make_model(str(tmp_path / "m"), TINY_A, seed=4, std=0.08)
    tokens = h.random_tokens(TINY_A, 12, seed=9)
    out = run_cli("run", d, "--tokens", ",".join(map(str, tokens)), "--max-tokens", "5", "--top-k", "3",
                  "--dtype", "float32", "--include-logits")
    assert out.returncode == 0, out.stderr[-2000:]
    res = json.loads(out.stdout)
    assert set(res) >= {"backend", "input_tokens", "next_token", "next_text", "generated_tokens", "generated_text",
                        "top_logits", "logit_count", "logits"}
    ref = plain.forward(TINY_A, h.read_weights(d), tokens)[-1]
    assert res["input_tokens"] == tokens and res["logit_count"] == 256 and len(res["logits"]) == 256
    assert res["next_token"] == int(ref.argmax()) == res["top_logits"][0]["token_id"]
    assert len(res["top_logits"]) == 3 and len(res["generated_tokens"]) == 5
    assert res["generated_tokens"][0] == res["next_token"]
    assert abs(res["top_logits"][0]["logit"] - float(ref.max())) < 1e-4

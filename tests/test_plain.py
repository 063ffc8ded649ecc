"""The plain implementation itself (CPU): pinned outputs, hand-computable cases, and properties
that hold by the formulas."""
import copy
import json
import math
import os

import pytest
import torch

import harness as h
import plain_llama4 as plain
from tiny_configs import TINY_A, TINY_B, TINY_C


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    base = tmp_path_factory.mktemp("plain")
    out = {}
    for name, cfg in (("A", TINY_A), ("B", TINY_B), ("C", TINY_C)):
        out[name] = (cfg, h.read_weights(h.make_model(str(base / name), cfg, seed=11, std=0.08)))
    return out


def test_pinned_outputs(models):
    golden = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "plain_tiny.json")))
    for name, (cfg, w) in models.items():
        g = golden[name]
        logits = plain.forward(cfg, w, g["tokens"])
        assert [int(r.argmax()) for r in logits] == g["argmax"]
        for p, row in g["rows"].items():
            assert torch.allclose(logits[int(p)][:12], torch.tensor(row), atol=2e-5), (name, p)
        assert abs(float(logits.double().abs().sum()) - g["checksum"]) < 1e-2 * max(1.0, g["checksum"] * 1e-3)


def test_rope_table_values():
    inv = plain.rope_inverse_frequencies(8, 10000.0, None)
    assert torch.allclose(inv, torch.tensor([1.0, 0.1, 0.01, 0.001]), rtol=1e-6)
    sc = dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=64)
    base = plain.rope_inverse_frequencies(32, 500000.0, None)
    got = plain.rope_inverse_frequencies(32, 500000.0, sc)
    for j in range(16):
        wavelen = 2 * math.pi / float(base[j])
        if wavelen > 64:
            want = float(base[j]) / 8
        elif wavelen < 16:
            want = float(base[j])
        else:
            s = (64 / wavelen - 1) / 3
            want = (1 - s) * float(base[j]) / 8 + s * float(base[j])
        assert abs(float(got[j]) - want) <= 1e-6 * want
    # all three branches occur in this table
    kinds = {("low" if 2 * math.pi / float(b) > 64 else "high" if 2 * math.pi / float(b) < 16 else "mid") for b in base}
    assert kinds == {"low", "high", "mid"}
    # Scout's factors (high == low) are a step; nothing is NaN
    scout = plain.rope_inverse_frequencies(128, 500000.0, dict(factor=16.0, low_freq_factor=1.0, high_freq_factor=1.0,
                                                               original_max_position_embeddings=8192))
    assert torch.isfinite(scout).all()


def test_rope_pairings_by_hand():
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0]]])
    inv = torch.tensor([math.pi / 2, math.pi])
    pos = torch.tensor([1])
    half = plain.apply_rope(x, pos, inv, interleaved=False)       # pairs (0,2), (1,3)
    assert torch.allclose(half, torch.tensor([[[-3.0, -2.0, 1.0, -4.0]]]), atol=1e-5)
    inter = plain.apply_rope(x, pos, inv, interleaved=True)       # pairs (0,1), (2,3)
    assert torch.allclose(inter, torch.tensor([[[-2.0, 1.0, -3.0, -4.0]]]), atol=1e-5)


def test_temperature_factor_by_hand():
    q = torch.ones(40, 1, 2)
    out = plain.attention_temperature(q, torch.arange(40), 16.0, 0.1)
    assert torch.allclose(out[:15], torch.ones(15, 1, 2))                       # pos + 1 < floor_scale
    assert torch.allclose(out[15, 0, 0], torch.tensor(1 + 0.1 * math.log(2.0)))   # pos 15: floor(16/16) = 1
    assert torch.allclose(out[31, 0, 0], torch.tensor(1 + 0.1 * math.log(3.0)))


def test_visibility_truth_table():
    vis = plain.visibility(7, 3)
    want = [[1, 0, 0, 0, 0, 0, 0], [1, 1, 0, 0, 0, 0, 0], [1, 1, 1, 0, 0, 0, 0], [0, 0, 0, 1, 0, 0, 0],
            [0, 0, 0, 1, 1, 0, 0], [0, 0, 0, 1, 1, 1, 0], [0, 0, 0, 0, 0, 0, 1]]
    assert vis.int().tolist() == want
    assert plain.visibility(4, None).int().tolist() == [[1, 0, 0, 0], [1, 1, 0, 0], [1, 1, 1, 0], [1, 1, 1, 1]]


def test_router_ties_and_scores():
    ids, scores = plain.router_top_k(torch.tensor([[0.5, 2.0, 2.0, -1.0, 2.0]]), 2)
    assert ids.tolist() == [[1, 2]] and torch.allclose(scores, torch.sigmoid(torch.tensor([[2.0, 2.0]])))


def test_score_scales_the_expert_input_not_its_output(models):
    cfg, w = models["A"]
    x = torch.randn(3, 64)
    p = "model.layers.0.feed_forward"
    out = plain.moe_feed_forward(plain.text_config(cfg), w, p, x)
    logits = x @ w[f"{p}.router.weight"].float().T
    ids, s = plain.router_top_k(logits, 1)
    shared = plain.swiglu(x, *(w[f"{p}.shared_expert.{n}_proj.weight"] for n in ("gate", "up", "down")))
    for t in range(3):
        e = int(ids[t, 0])
        ws = [w[f"{p}.experts.{n}_proj.weight"][e] for n in ("gate", "up", "down")]
        scaled_in = plain.swiglu(x[t:t + 1] * s[t, 0], *ws)[0]
        scaled_out = plain.swiglu(x[t:t + 1], *ws)[0] * s[t, 0]
        assert torch.allclose(out[t] - shared[t], scaled_in, atol=1e-6)
        assert not torch.allclose(scaled_in, scaled_out, atol=1e-4)


def test_properties_of_the_layer_kinds(models):
    cfg, w = models["A"]
    toks = h.random_tokens(cfg, 30, seed=2)
    # a chunk at least as long as the sequence is plain causal attention
    big = copy.deepcopy(cfg); big["attention_chunk_size"] = 64
    all_global = copy.deepcopy(big); all_global["attention_chunk_size"] = 10 ** 6
    assert torch.allclose(plain.forward(big, w, toks), plain.forward(all_global, w, toks), atol=1e-6)
    # within the first chunk and below floor_scale the chunk rule and the temperature change nothing
    short = toks[:15]
    off = copy.deepcopy(cfg); off["attn_temperature_tuning"] = False; off["attention_chunk_size"] = 15
    assert torch.allclose(plain.forward(cfg, w, short), plain.forward(off, w, short), atol=1e-6)
    # ... and beyond them they do
    assert not torch.allclose(plain.forward(cfg, w, toks + toks), plain.forward(off, w, toks + toks), atol=1e-4)
    # logits at a position do not depend on later tokens
    full = plain.forward(cfg, w, toks)
    assert torch.allclose(plain.forward(cfg, w, toks[:11]), full[:11], atol=1e-5)


def test_what_the_layer_kinds_take_from_positions(models):
    """A NoPE layer without temperature takes nothing from absolute positions; a rotary layer only
    differences of positions (all of the sequence within one chunk); with temperature the NoPE layer
    does change once floor((pos + 1) / floor_scale) moves."""
    cfg, w = models["A"]
    c = plain.text_config(copy.deepcopy(cfg))
    c["attention_chunk_size"] = 4096
    x = torch.randn(20, c["hidden_size"], generator=torch.Generator().manual_seed(3))
    inv = plain.rope_inverse_frequencies(c["head_dim"], c["rope_theta"], c.get("rope_scaling"))
    rotary, nope = "model.layers.0.self_attn", "model.layers.1.self_attn"
    assert plain.layer_uses_rope(c, 0) and not plain.layer_uses_rope(c, 1)
    no_temp = dict(c, attn_temperature_tuning=False)
    a0 = plain.attention(no_temp, w, nope, 1, x, inv)
    assert torch.allclose(a0, plain.attention(no_temp, w, nope, 1, x, inv, first_position=1000), atol=1e-6)
    r0 = plain.attention(c, w, rotary, 0, x, inv)
    assert torch.allclose(r0, plain.attention(c, w, rotary, 0, x, inv, first_position=777), atol=2e-5)
    assert not torch.allclose(r0, plain.attention(dict(c, attention_chunk_size=8), w, rotary, 0, x, inv), atol=1e-4)
    t0 = plain.attention(c, w, nope, 1, x[:10], inv)                                    # positions 0..9: factor 1
    assert torch.allclose(t0, plain.attention(no_temp, w, nope, 1, x[:10], inv), atol=1e-6)
    assert not torch.allclose(t0, plain.attention(c, w, nope, 1, x[:10], inv, first_position=160), atol=1e-4)


def test_one_expert_of_one_is_a_dense_layer_with_a_scaled_input(models):
    """k = 1 of E = 1: the routed part is the dense feed-forward of the expert's weights on the input
    scaled by sigmoid(x . w_router), and the shared expert's dense feed-forward is added."""
    cfg, w = models["A"]
    c = plain.text_config(cfg)
    p = "model.layers.0.feed_forward"
    one = {k: (v[:1] if ".experts." in k or k.endswith("router.weight") else v) for k, v in w.items() if k.startswith(p)}
    x = torch.randn(9, c["hidden_size"], generator=torch.Generator().manual_seed(4))
    out = plain.moe_feed_forward(dict(c, num_local_experts=1, num_experts_per_tok=1), one, p, x)
    score = torch.sigmoid(x @ one[f"{p}.router.weight"].float().T)                       # [9, 1]
    dense = {f"d.{n}_proj.weight": one[f"{p}.experts.{n}_proj.weight"][0] for n in ("gate", "up", "down")}
    shared = {f"s.{n}_proj.weight": one[f"{p}.shared_expert.{n}_proj.weight"] for n in ("gate", "up", "down")}
    want = plain.dense_feed_forward(dense, "d", x * score) + plain.dense_feed_forward(shared, "s", x)
    assert torch.allclose(out, want, atol=1e-6)


def test_sampler_follows_the_reference(models):
    logits = torch.tensor([0.2, 0.1, 4.0, 3.0, 2.0])
    assert plain.sample(logits, 0.0, 1.0, 0, 0.3) == 2
    assert plain.sample(torch.tensor([1.0, 3.0, 3.0]), 0.0, 1.0, 0, 0.0) == 1       # tie -> lower id
    # temperature only: inverse CDF in vocabulary order
    p = torch.softmax(logits, 0)
    cum = torch.cumsum(p, 0)
    for u in (0.0, 0.01, 0.3, 0.7, 0.99):
        assert plain.sample(logits, 1.0, 1.0, 0, u) == int((cum > u).nonzero()[0])
    # ranked: top_p 0.8 keeps tokens 2, 3 (0.647 + 0.238); the walk is in descending order
    assert plain.sample(logits, 1.0, 0.8, 0, 0.5) == 2 and plain.sample(logits, 1.0, 0.8, 0, 0.95) == 3
    assert plain.sample(logits, 1.0, 0.9, 0, 0.95) == 4                               # 0.9 needs a third token
    assert plain.sample(logits, 1.0, 1.0, 1, 0.99) == 2                               # top-k 1
    # the generator: first draws for seed 42 are fixed by the recurrence
    g = plain.Lcg(42)
    state = (42 ^ 0x9E3779B97F4A7C15) & (2 ** 64 - 1)
    state = (state * 6364136223846793005 + 1442695040888963407) % 2 ** 64
    assert g.next_f32() == (state >> 40) / 2 ** 24

"""The engine at the layer sizes it is benchmarked at: two-layer models with Scout's and with
Maverick's matrices (hidden 5120, 40 heads over 8 kv heads of 128, experts of 8192, a vocabulary
of 202,048), one rotary chunked layer and one global NoPE layer with temperature, weights made
on the device from a seed. A plain model of this size cannot be run on the CPU in a test's
time, so the checks are between the engine's own paths, whose kernels differ: the float32 path
(plain SIMT kernels, true 32-bit library products) under every way of cutting against itself
whole, within the float32 tolerance, which a single wrong page breaks; and the bfloat16 path
(tcgen05 grouped products and attention, TMA decode attention, weight-streaming expert kernels,
captured decode steps) against the float32 path given the bfloat16 run's expert choices, at spot
rows around every edge. Prompts cross position 8,192 (Scout's chunk and temperature floor) in a
portion, between portions and while decoding; in the mixed regime the chunked pool is a few pages
larger than one chunk, so the pages of the dead chunk come round again.
(The reference checks its served model against its float32 forward in the same manner:
crates/hi-cuda/src/lib.rs:24889-24981.)"""
import gc

import numpy as np
import pytest
import torch

import harness as h

pytestmark = pytest.mark.gpu

PAGE = 64
LAYER_SIZES = {
    "architectures": ["Llama4ForCausalLM"], "model_type": "llama4_text",
    "vocab_size": 202048, "hidden_size": 5120, "num_hidden_layers": 2,
    "num_attention_heads": 40, "num_key_value_heads": 8, "head_dim": 128, "rms_norm_eps": 1e-5,
    "rope_theta": 500000.0, "no_rope_layers": [1, 0],
    "attn_temperature_tuning": True, "attn_scale": 0.1,
    "num_experts_per_tok": 1, "intermediate_size": 8192, "intermediate_size_mlp": 16384,
    "tie_word_embeddings": False, "max_position_embeddings": 262144,
}
SCOUT = dict(LAYER_SIZES, attention_chunk_size=8192, floor_scale=8192, use_qk_norm=True, interleave_moe_layer_step=1,
             num_local_experts=16,
             rope_scaling={"rope_type": "llama3", "factor": 16.0, "low_freq_factor": 1.0, "high_freq_factor": 1.0,
                           "original_max_position_embeddings": 8192})
# Maverick's matrices: a dense layer of 16,384 and a layer of 128 experts; the chunk and the temperature
# floor are set to 1,024 here so that a 2,100-token request crosses both twice
MAVERICK = dict(LAYER_SIZES, attention_chunk_size=1024, floor_scale=1024, use_qk_norm=False, interleave_moe_layer_step=2,
                num_local_experts=128, rope_scaling=None)


def schedule(plan, max_live=4):
    """A mixed trace from a plan {request: (tokens, prompt length, portion sizes, first step)}: in
    every step each live request feeds its next portion, or one token once its prompt is in."""
    waiting = sorted(plan, key=lambda r: plan[r][3])
    live, done, steps, t = [], {}, [], 0
    turn = {r: 0 for r in plan}
    while waiting or live:
        while waiting and len(live) < max_live and plan[waiting[0]][3] <= t:
            live.append(waiting.pop(0))
        entries, end = [], []
        for rid in list(live):
            toks, prompt, sizes, _ = plan[rid]
            at = done.get(rid, 0)
            n = min(sizes[turn[rid] % len(sizes)], prompt - at) if at < prompt else 1
            turn[rid] += 1
            entries.append((rid, toks[at:at + n], list(range(n))))
            done[rid] = at + n
            if done[rid] == len(toks):
                end.append(rid)
                live.remove(rid)
        if entries:
            steps.append((entries, end))
        t += 1
    return steps


def keep_spots(steps, spots):
    """Logits only where they are compared: portions keep the positions named in ``spots``, single
    tokens keep theirs (a step of single tokens that all want their logits is what is captured)."""
    at, out = {}, []
    for entries, end in steps:
        new = []
        for rid, toks, want in entries:
            start = at.get(rid, 0)
            if len(toks) > 1:
                want = [w for w in want if start + w in spots[rid]]
            new.append((rid, toks, want))
            at[rid] = start + len(toks)
        out.append((new, end))
    return out


def compare(got, want, tol, what):
    for rid, rows in got.items():
        scale = max(float(np.abs(r).max()) for r in want[rid].values())
        for p in sorted(rows):
            err = float(np.abs(rows[p] - want[rid][p]).max()) / scale
            assert np.isfinite(err) and err <= tol, f"{what}: request {rid!r} first differs at position {p}: rel err {err:.3e} > {tol:.1e}"


def release(engine):
    del engine
    gc.collect()
    torch.cuda.empty_cache()


def run_model(cfg, seed, requests, traces, pools, expect_kernels):
    """bfloat16 under every trace (with the routers' choices recorded), then float32: whole, every
    trace unforced against whole, and whole given each bfloat16 run's choices against that run."""
    from hi_b200.engine.core import Engine
    from hi_b200.kernels import ops

    options = dict(kv_page_size=PAGE, kv_cache_tokens=pools[0] * PAGE, windowed_cache_tokens=pools[1] * PAGE,
                   max_active_requests=4)
    spots_all = {rid: set(range(len(t))) for rid, t in requests.items()}
    whole = h.trace_whole(requests)
    bf16 = {}
    before = dict(ops.CALLS)
    eng = Engine.from_config(cfg, seed=seed, std=0.02, dtype="bfloat16", **options)
    for name, steps in traces.items():
        got, routing = h.replay_in_process(eng, steps, record_routing=True)
        bf16[name] = (got, routing)
        assert not eng.manager.requests and all(p.free == p.total for p in eng.manager.pools), f"bfloat16 {name}: pages lost"
    ran = {k for k, v in ops.CALLS.items() if v > before.get(k, 0)}
    assert expect_kernels <= ran, f"bfloat16: {sorted(expect_kernels - ran)} did not run (ran: {sorted(ran)})"
    assert eng._graphs, "no decode step was captured"
    snap = eng.manager.snapshot()
    release(eng)

    eng = Engine.from_config(cfg, seed=seed, std=0.02, dtype="float32", **options)
    spots = {rid: set() for rid in requests}
    for name, (got, _r) in bf16.items():
        for rid, rows in got.items():
            spots[rid] |= set(rows)
    reference, own = h.replay_in_process(eng, keep_spots(whole, spots), record_routing=True)
    for name, steps in traces.items():
        got, _ = h.replay_in_process(eng, steps)
        compare(got, reference, h.TOL_F32, f"float32 {name} against float32 whole")
        assert not eng.manager.requests and all(p.free == p.total for p in eng.manager.pools), f"float32 {name}: pages lost"
    flips = 0
    for name, (got, routing) in bf16.items():
        live = {rid: toks for rid, toks in requests.items() if rid in got}
        given, _ = h.replay_in_process(eng, keep_spots(h.trace_whole(live), spots), forced_routing=routing)
        compare(got, given, h.TOL_BF16, f"bfloat16 {name} against float32 given its expert choices")
        for rid in live:
            for layer, ids in routing[rid].items():
                flips += int((ids.long().sort(-1).values != own[rid][layer].long().sort(-1).values).any(-1).sum())
    total = sum(len(t) for t in requests.values()) * len(traces)
    assert flips <= 0.05 * total, f"bfloat16 picked another expert than float32 for {flips} of about {total} tokens"
    release(eng)
    return snap


def test_scout_sized_layers_across_the_chunk_edge():
    cfg = SCOUT
    lengths = {"a": 8250, "b": 300, "c": 700, "d": 200}
    reqs = {rid: h.random_tokens(cfg, n, seed=900 + i) for i, (rid, n) in enumerate(lengths.items())}
    edge = {0, 1, 2999, 3000, 3001, 8149, 8150, 8187, 8188, 8190, 8191, 8192, 8193, 8196, 8197, 8249}
    spots = {"a": edge, "b": {0, 259, 299}, "c": {0, 1, 649, 699}, "d": {0, 149, 199}}
    alone = {"a": reqs["a"]}
    traces = {
        "whole": keep_spots(h.trace_whole({"a": reqs["a"], "c": reqs["c"]}), spots),
        # 8,150 tokens in one step, then one by one over position 8,192
        "tail": keep_spots(h.trace_tail_decode(alone, tail=100), spots),
        # a portion that ends on the chunk's last page, one that crosses 8,192, two tokens, one token
        "portions": keep_spots(h.trace_portions(alone, sizes=(3000, 2, 2600, 1, 2500, 85, 9, 2, 51)), spots),
        # a, b and c together; a crosses 8,192 while decoding; d starts once a's dead chunk is back in the pool
        "mixed": keep_spots(schedule({"a": (reqs["a"], 8150, (3000, 3000, 1000, 1000, 150), 0),
                                      "b": (reqs["b"], 260, (260,), 0), "c": (reqs["c"], 650, (400, 250), 1),
                                      "d": (reqs["d"], 150, (2, 148), 60)}), spots),
    }
    assert max(len(e) for e, _ in traces["mixed"]) >= 3
    # all keys: 129 + 5 + 11 + 4 pages; chunked: a's chunk (128) + b (5) + c (11) + the page a writes past the edge + 2
    snap = run_model(cfg, 3, reqs, traces, pools=(150, 147),
                     expect_kernels={"attention_prefill_tc", "attention_decode_tma", "attention_decode_fused", "moe_gate_up_tc", "moe_down_tc",
                                     "moe_gate_up", "moe_down", "router_plan"})
    chunked = [g for g in snap["groups"] if g["window"]][0]
    assert chunked["allocations"] > chunked["total"], "the dead chunk's pages were not used again"
    assert chunked["peak"] <= 147


def test_maverick_sized_layers_with_128_experts():
    cfg = MAVERICK
    lengths = {"a": 2100, "b": 500, "c": 300, "d": 150}
    reqs = {rid: h.random_tokens(cfg, n, seed=950 + i) for i, (rid, n) in enumerate(lengths.items())}
    spots = {"a": {0, 1, 1022, 1023, 1024, 1025, 2047, 2048, 2049, 2059, 2099}, "b": {0, 459, 499},
             "c": {0, 269, 299}, "d": {0, 99, 149}}
    alone = {"a": reqs["a"]}
    traces = {
        "whole": keep_spots(h.trace_whole({"a": reqs["a"], "b": reqs["b"]}), spots),
        "tail": keep_spots(h.trace_tail_decode(alone, tail=60), spots),      # decodes over position 2,048
        "portions": keep_spots(h.trace_portions(alone, sizes=(1000, 2, 30, 1, 900, 140, 27)), spots),
        "mixed": keep_spots(schedule({"a": (reqs["a"], 2040, (700, 700, 600, 40), 0), "b": (reqs["b"], 460, (460,), 0),
                                      "c": (reqs["c"], 270, (135, 135), 1), "d": (reqs["d"], 100, (2, 98), 30)}), spots),
    }
    # chunked pool: a's chunk (16 pages) + its next page + b (8) + c (5) + d (3) + 2
    snap = run_model(cfg, 4, reqs, traces, pools=(52, 35),
                     expect_kernels={"attention_prefill_tc", "attention_decode_tma", "attention_decode_fused", "moe_gate_up_tc", "moe_down_tc",
                                     "moe_gate_up", "moe_down", "router_plan"})
    chunked = [g for g in snap["groups"] if g["window"]][0]
    assert chunked["allocations"] > chunked["total"], "dead chunks' pages were not used again"

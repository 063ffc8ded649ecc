"""Configurations drawn at random (seeded): every size and option of the architecture moves at
once, small odd widths as well as sizes at which the tensor-core kernels take over, and each
draw goes through the four ways of cutting against the plain model, in 32-bit and in bfloat16."""
import random

import pytest

import harness as h

pytestmark = pytest.mark.gpu


def draw(rng: random.Random, large: bool) -> dict:
    nkv = rng.choice([1, 2, 3, 4, 5])
    nh = nkv * rng.choice([1, 2, 3, 4, 5, 7, 8])
    experts = rng.choice([2, 4, 5, 8, 16]) if large else rng.randrange(1, 10)
    cfg = {
        "architectures": ["Llama4ForCausalLM"], "model_type": "llama4_text",
        "vocab_size": rng.randrange(90, 1200),
        "hidden_size": rng.choice([256, 320, 384, 448, 512, 576]) if large else rng.choice([2, 4, 8, 16]) * rng.randrange(3, 30),
        "num_hidden_layers": rng.randrange(1, 5),
        "num_attention_heads": nh, "num_key_value_heads": nkv,
        "head_dim": rng.choice([32, 64, 64, 128, 128, 256]) if large else rng.choice([16, 32, 48, 64, 80, 96, 112, 128]),
        "rms_norm_eps": rng.choice([1e-5, 1e-6, 3e-4]), "rope_theta": rng.choice([10000.0, 500000.0]),
        "rope_scaling": rng.choice([None, {"rope_type": "llama3", "factor": rng.choice([4.0, 8.0, 16.0]),
                                           "low_freq_factor": 1.0, "high_freq_factor": rng.choice([1.0, 4.0]),
                                           "original_max_position_embeddings": rng.choice([32, 64, 128])}]),
        "attention_chunk_size": rng.choice([64, 128, 192, 256, 320]) if large else rng.choice([8, 16, 24, 40, 64, 100, 128, 192]),
        "nope_layer_interval": rng.choice([1, 2, 3, 4]),
        "use_qk_norm": rng.random() < 0.6, "attn_temperature_tuning": rng.random() < 0.6,
        "floor_scale": rng.choice([8, 16, 32, 100]), "attn_scale": rng.choice([0.1, 0.25]),
        "interleave_moe_layer_step": rng.choice([1, 1, 2, 3]),
        "num_local_experts": experts, "num_experts_per_tok": rng.randrange(1, min(experts, 3) + 1),
        "intermediate_size": rng.choice([128, 192, 256, 320]) if large else rng.choice([2, 8, 16]) * rng.randrange(3, 20),
        "intermediate_size_mlp": rng.choice([256, 384, 512]) if large else rng.choice([2, 8, 16]) * rng.randrange(3, 30),
        "tie_word_embeddings": rng.random() < 0.3, "max_position_embeddings": 4096,
    }
    if rng.random() < 0.3:
        cfg["rope_interleaved"] = True
    return cfg


@pytest.mark.parametrize("seed,large", [(1, False), (5, False), (7, False), (9, False), (47, False),
                                        (203, True), (207, True), (211, True)])
def test_a_random_configuration_in_the_four_ways_of_cutting(seed, large, tmp_path):
    from hi_b200.engine.core import Engine

    rng = random.Random(seed)
    cfg = draw(rng, large)
    page = rng.choice([16, 32, 64, 64, 128]) if large else rng.choice([4, 8, 16, 64])
    lengths = [rng.randrange(3, 60), rng.randrange(20, 120), rng.randrange(60, 200)] + \
        ([rng.randrange(200, 520), rng.randrange(130, 300)] if large else [rng.randrange(40, 260)])
    mdir = h.make_model(str(tmp_path / "m"), cfg, seed=seed, std=0.04 if large else 0.08)
    weights = h.read_weights(mdir)
    reqs = {f"r{i}": h.random_tokens(cfg, n, seed=seed * 10 + i) for i, n in enumerate(lengths)}
    rounded = lambda n: -(-n // page) * page
    cap = max(rounded(n) for n in lengths) + 2 * page
    mixed_cap = max(cap, sum(sorted(rounded(n) for n in lengths)[-2:]) + page)
    for dtype, tol in (("float32", h.TOL_F32), ("bfloat16", h.TOL_BF16)):
        for regime, steps, tokens in (("whole", h.trace_whole(reqs), cap), ("tail", h.trace_tail_decode(reqs), cap),
                                      ("portions", h.trace_portions(reqs), cap),
                                      ("mixed", h.trace_mixed(reqs, max_tokens=mixed_cap, page=page, seed=seed), mixed_cap)):
            eng = Engine.from_dir(mdir, dtype=dtype, kv_page_size=page, kv_cache_tokens=tokens,
                                  max_active_requests=4, debug_poison=True)
            got, forced = h.replay_in_process(eng, steps, record_routing=(dtype == "bfloat16"))
            h.compare_with_plain(cfg, weights, reqs, got, tol, forced=forced if dtype == "bfloat16" else None,
                                 what=f"seed {seed} {cfg} page {page}: {dtype} {regime}", margin=h.ROUTING_MARGIN)
            assert not eng.manager.requests
            for pool in eng.manager.pools:
                assert pool.free == pool.total, "pages were lost"

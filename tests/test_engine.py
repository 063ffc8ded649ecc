"""The engine in process, with small pages so that every edge is crossed often: the four ways
of cutting, long decoding, the first tokens, crafted weights that make one far key or one page
matter, a schedule that runs a layer twice, generation through the entry point, and toy parts
registered from here: a mixer with state of its own, a position encoding that is no rotation and
a feed-forward with routing."""
import math

import numpy as np
import pytest
import torch

import harness as h
import plain_llama4 as plain
from tiny_configs import TINY_A, TINY_B, TINY_C

pytestmark = pytest.mark.gpu

DTYPES = [("float32", h.TOL_F32), ("bfloat16", h.TOL_BF16)]


def engine_for(mdir, dtype, page, tokens=256, slots=4, **kw):
    from hi_b200.engine.core import Engine

    return Engine.from_dir(mdir, dtype=dtype, kv_page_size=page, kv_cache_tokens=tokens, max_active_requests=slots, **kw)


def check(cfg, mdir, dtype, tol, steps, reqs, page, tokens, what, **kw):
    eng = engine_for(mdir, dtype, page, tokens, **kw)
    got, forced = h.replay_in_process(eng, steps, record_routing=(dtype == "bfloat16"))
    h.compare_with_plain(cfg, h.read_weights(mdir), reqs, got, tol, forced=forced if dtype == "bfloat16" else None,
                         what=what, margin=h.ROUTING_MARGIN)
    assert not eng.manager.requests, "requests left open"
    for pool in eng.manager.pools:
        assert pool.free == pool.total, "pages were lost"
    return eng


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("name,page", [("A", 4), ("B", 16), ("C", 8), ("D", 16), ("D", 64)])
def test_four_ways_of_cutting(name, page, dtype, tol, model_dirs):
    cfg, mdir = model_dirs[name]
    reqs = {f"r{i}": h.random_tokens(cfg, n, seed=7 + i) for i, n in enumerate([23, 35, 49, 64, 97, 70])}
    small = max(128, 2 * page)
    mixed_cap = max(288, 5 * page)
    for regime, steps, cap in (("whole", h.trace_whole(reqs), small), ("tail", h.trace_tail_decode(reqs), small),
                               ("portions", h.trace_portions(reqs), small),
                               ("mixed", h.trace_mixed(reqs, max_tokens=mixed_cap, page=page, seed=5), mixed_cap)):
        eng = check(cfg, mdir, dtype, tol, steps, reqs, page, cap, f"{name} {dtype} page {page} {regime}",
                    debug_poison=True)
        if regime == "mixed" and page <= 16:
            snap = eng.manager.snapshot()
            assert all(g["allocations"] > g["total"] for g in snap["groups"]), "pages were not used again"


@pytest.mark.parametrize("dtype,tol", DTYPES)
def test_long_decoding_and_first_tokens(dtype, tol, model_dirs):
    """A 5-token prompt fed one token at a time from position 0, then 300 decoded tokens one by one:
    many chunk edges, many pages freed and used again by the same request."""
    cfg, mdir = model_dirs["A"]
    toks = h.random_tokens(cfg, 305, seed=21)
    steps = [([("x", [t], [0])], []) for t in toks]
    steps[-1] = (steps[-1][0], ["x"])
    eng = check(cfg, mdir, dtype, tol, steps, {"x": toks}, 8, 352, f"long decode {dtype}", debug_poison=True)
    chunked = [g for g in eng.manager.snapshot()["groups"] if g["window"]]
    assert chunked and chunked[0]["peak"] <= 32 // 8 + 1, "the chunked group kept pages of dead chunks"


def peaky_overrides(cfg, mdir, scale=6.0):
    """q and k projections scaled up: softmax is then far from uniform, so a key that is missing,
    stale or at the wrong place changes the logits far beyond the tolerance."""
    w = h.read_weights(mdir)
    return {n: (t.float() * scale) for n, t in w.items() if n.endswith(("q_proj.weight", "k_proj.weight"))}


# how far q and k can be scaled up before the oracle's own float32 rounding (measured against
# float64 in the test) or bfloat16's three digits drown the comparison. A and C norm q and k on
# their rotary layers, so the sharpening lands on the global layers (every earlier key, with
# temperature); B has no such norm, its scores grow with the square of the scale and its float32
# oracle loses five digits at scale 2, so it is left out here.
SHARPEN = {("A", "float32"): 4.0, ("A", "bfloat16"): 2.5, ("C", "float32"): 2.0, ("C", "bfloat16"): 2.0}


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("name", ["A", "C"])
def test_peaked_attention_under_cutting(name, dtype, tol, model_dirs, tmp_path):
    cfg, mdir = model_dirs[name]
    sharp = h.make_model(str(tmp_path / "sharp"), cfg, seed=11, std=0.08,
                         overrides=peaky_overrides(cfg, mdir, SHARPEN[name, dtype]))
    reqs = {f"r{i}": h.random_tokens(cfg, n, seed=40 + i) for i, n in enumerate([130, 75, 48])}
    w = h.read_weights(sharp)
    ref32 = plain.forward(cfg, w, reqs["r0"])
    with plain.precision(torch.float64):
        ref64 = plain.forward(cfg, {k: v.double() for k, v in w.items()}, reqs["r0"])
    assert h.rel_err(ref32, ref64.float()) < h.TOL_F32 / 4, "the sharpened model is too ill-conditioned to be an oracle"
    for steps, regime in ((h.trace_portions(reqs), "portions"), (h.trace_mixed(reqs, 272, 16, seed=9), "mixed")):
        check(cfg, sharp, dtype, tol, steps, reqs, 16, 272, f"peaked {name} {dtype} {regime}", debug_poison=True)


def test_schedule_runs_a_layer_twice(model_dirs):
    """The order of layers is data: layer 0 runs twice (two cache slots), then layer 1."""
    from hi_b200.config.registry import load_architecture
    from hi_b200.engine.core import Engine, parse_dtype
    from hi_b200.parts.model import Model
    from hi_b200.parts.spec import ModelSpec, ScheduleEntry
    from hi_b200.weights.loader import load_from_dir
    import dataclasses

    dtype, tol = "float32", h.TOL_F32
    cfg, mdir = model_dirs["A"]
    arch, typed, _ = load_architecture(mdir)
    spec = arch.build_spec(typed)
    order = [0, 1, 0, 1, 1]
    spec = dataclasses.replace(spec, schedule=tuple(ScheduleEntry(layer=l, cache=i) for i, l in enumerate(order)))
    model = Model(spec, parse_dtype(dtype), "cuda:0")
    load_from_dir(model, mdir, arch.normalize_tensor_name)
    eng = Engine(model, kv_page_size=8, kv_cache_tokens=128, max_active_requests=2)
    toks = h.random_tokens(cfg, 90, seed=3)
    steps = h.trace_portions({"a": toks})
    got, _ = h.replay_in_process(eng, steps, record_routing=False)
    ref = plain.forward(cfg, h.read_weights(mdir), toks, schedule=order)
    out = torch.tensor(np.stack([got["a"][p] for p in range(len(toks))]))
    err = h.rel_err(out, ref)
    assert err <= tol, f"repeated layers: rel err {err}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(dtype, model_dirs):
    """hi_b200.generate: greedy tokens of four prompts, batched by the scheduler, against the plain
    model fed the same tokens: every generated token must be (within rounding) the plain argmax."""
    import hi_b200

    cfg, mdir = model_dirs["A"]
    w = h.read_weights(mdir)
    prompts = [h.random_tokens(cfg, n, seed=60 + n) for n in (7, 19, 33, 48)]
    outs = hi_b200.generate(mdir, prompts, hi_b200.SamplingParams(max_tokens=16, ignore_eos=True), dtype=dtype,
                            kv_page_size=16, max_batched_tokens=40, max_batch_size=4, kv_cache_tokens=512)
    slack = 1e-4 if dtype == "float32" else 0.08
    for prompt, out in zip(prompts, outs):
        assert out.completion_tokens == 16 and out.finish_reason == "length"
        ref = plain.forward(cfg, w, prompt + out.token_ids)
        for i, tok in enumerate(out.token_ids):
            row = ref[len(prompt) - 1 + i]
            assert float(row.max() - row[tok]) <= slack * float(row.abs().max()), (
                f"{dtype}: generated token {i} = {tok} is not the plain argmax {int(row.argmax())}")
        if dtype == "float32":
            assert out.token_ids == [int(ref[len(prompt) - 1 + i].argmax()) for i in range(16)]


def test_seeded_sampling_does_not_depend_on_batching(model_dirs):
    import hi_b200

    cfg, mdir = model_dirs["B"]
    prompts = [h.random_tokens(cfg, n, seed=80 + n) for n in (5, 40, 70)]
    sp = [hi_b200.SamplingParams(max_tokens=12, temperature=0.9, seed=5 + i, ignore_eos=True) for i in range(3)]
    llm = hi_b200.LLM(mdir, dtype="float32", kv_page_size=16, max_batch_size=4, kv_cache_tokens=512)
    together = [o.token_ids for o in llm.generate(prompts, sp)]
    alone = [llm.generate([p], [s])[0].token_ids for p, s in zip(prompts, sp)]
    assert together == alone


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_launching_a_step_ahead_changes_no_token(dtype, model_dirs):
    """With lookahead a decode step is launched before the host has read the tokens of the step
    before it (they are fed on the device), requests that stop leave an unread row in the step
    already launched, and rows ranked on the host make their step wait: the generated tokens, the
    reasons and the streamed tokens are those of the step-by-step loop. The stop token is chosen
    from what the model really generates, so that requests end in the middle."""
    import hi_b200

    cfg, mdir = model_dirs["B"]
    prompts = [h.random_tokens(cfg, n, seed=70 + n) for n in (9, 30, 3, 44, 17)]

    def params(stop):
        return [hi_b200.SamplingParams(max_tokens=24, temperature=0.0 if i % 2 else 0.9, seed=11 + i, ignore_eos=True,
                                       stop_token_ids=stop, top_k=5 if i == 4 else None) for i in range(5)]

    free = hi_b200.LLM(mdir, dtype=dtype, kv_page_size=16, max_batch_size=3, kv_cache_tokens=1024, lookahead=False)
    seen = [o.token_ids for o in free.generate(prompts, params(()))]
    stop = tuple({out[len(out) // 2] for out in seen[:3]})          # tokens that do occur half-way
    runs = []
    for ahead in (False, True):
        llm = hi_b200.LLM(mdir, dtype=dtype, kv_page_size=16, max_batch_size=3, kv_cache_tokens=1024, lookahead=ahead)
        streamed = {}
        outs = llm.generate(prompts, params(stop), on_token=lambda rid, tok: streamed.setdefault(rid, []).append(tok))
        assert all(streamed.get(o.request_id, []) == o.token_ids for o in outs)
        assert not llm.engine.manager.requests and all(p.free == p.total for p in llm.engine.manager.pools)
        runs.append([(o.token_ids, o.finish_reason) for o in outs])
    assert runs[0] == runs[1]
    assert any(reason == "stop" and len(toks) < 24 for toks, reason in runs[0]), "no request stopped in the middle"
    # and ahead in a pool so small that requests are preempted while a step of theirs is in flight
    tight = hi_b200.LLM(mdir, dtype=dtype, kv_page_size=16, max_batch_size=3, kv_cache_tokens=96, windowed_cache_tokens=96,
                        lookahead=True)
    outs = tight.generate(prompts, params(stop))
    assert [(o.token_ids, o.finish_reason) for o in outs] == runs[0]
    assert sum(o.preemptions for o in outs) >= 1, "the pool was large enough: nothing was preempted"
    tight.engine.manager.check_invariants()
    assert not tight.engine.manager.requests and all(p.free == p.total for p in tight.engine.manager.pools)


def test_generation_with_so_few_pages_that_requests_are_preempted(model_dirs):
    """Four requests in a cache that cannot hold them all to the end: decoding runs out of pages,
    the scheduler preempts the youngest request (its pages go back, it is computed again from its
    prompt and the tokens it had generated), and every request still ends with exactly the tokens
    it generates alone: greedy, and sampled with a seed (the generator's state survives)."""
    import hi_b200

    cfg, mdir = model_dirs["A"]
    prompts = [h.random_tokens(cfg, n, seed=90 + n) for n in (30, 26, 21, 17)]
    for sp in ([hi_b200.SamplingParams(max_tokens=40, ignore_eos=True)] * 4,
               [hi_b200.SamplingParams(max_tokens=40, temperature=0.8, seed=3 + i, ignore_eos=True) for i in range(4)]):
        roomy = hi_b200.LLM(mdir, dtype="float32", kv_page_size=8, max_batch_size=4, kv_cache_tokens=1024)
        alone = [roomy.generate([p], [s])[0].token_ids for p, s in zip(prompts, sp)]
        tight = hi_b200.LLM(mdir, dtype="float32", kv_page_size=8, max_batch_size=4, kv_cache_tokens=176,
                            windowed_cache_tokens=176)
        outs = tight.generate(prompts, sp)
        assert sum(o.preemptions for o in outs) >= 1, "the pool was large enough: nothing was preempted"
        assert [o.token_ids for o in outs] == alone
        assert all(o.finish_reason == "length" and o.completion_tokens == 40 for o in outs)
        tight.engine.manager.check_invariants()
        assert not tight.engine.manager.requests and all(p.free == p.total for p in tight.engine.manager.pools)


def test_abort_frees_everything_also_with_a_step_in_flight(model_dirs):
    """abort() between calls of step(), while a step launched ahead still holds a row of the request:
    its pages and slot are back at once, the row is computed for nobody, a waiting request is
    dropped without ever running, and the others end with the tokens they generate alone."""
    import hi_b200

    cfg, mdir = model_dirs["A"]
    prompts = [h.random_tokens(cfg, n, seed=120 + n) for n in (14, 22, 9, 30)]
    sp = hi_b200.SamplingParams(max_tokens=24, ignore_eos=True)
    alone = [hi_b200.LLM(mdir, dtype="float32", kv_page_size=8, kv_cache_tokens=512).generate([p], sp)[0].token_ids
             for p in prompts]
    llm = hi_b200.LLM(mdir, dtype="float32", kv_page_size=8, max_batch_size=3, kv_cache_tokens=512, lookahead=True)
    reqs = [llm.add_request(p, sp, request_id=f"r{i}") for i, p in enumerate(prompts)]
    for _ in range(6):
        llm.step()
    assert llm._launched is not None and "r1" in llm._launched.row_of, "no step of r1 is in flight"
    assert reqs[3].status == "waiting"
    llm.abort("r3")
    llm.abort("r1")
    assert reqs[1].status == "finished" and reqs[1].finish_reason == "aborted" and reqs[3].finish_reason == "aborted"
    assert not llm.engine.manager.is_open("r1") and reqs[3].output == []
    llm.engine.manager.check_invariants()
    kept = len(reqs[1].output)
    while any(r.status != "finished" for r in reqs):
        llm.step()
    llm.step()                                                    # the last launched step is read
    assert len(reqs[1].output) == kept and reqs[1].output == alone[1][:kept]
    assert reqs[0].output == alone[0] and reqs[2].output == alone[2]
    llm.engine.manager.check_invariants()
    assert not llm.engine.manager.requests and all(p.free == p.total for p in llm.engine.manager.pools)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_weights_generated_on_the_device_are_the_folders_weights(dtype, tmp_path):
    """Engine.from_config(seed) (weights made by a kernel on the device) and
    Engine.from_dir(write_random_model(seed)) (the same numbers made on the host and stored) are
    the same model: equal weights, and logits equal bit for bit."""
    from hi_b200.engine.core import Engine, StepEntry
    from hi_b200.weights import write_random_model

    cfg = TINY_C
    mdir = write_random_model(cfg, str(tmp_path / "m"), seed=77, std=0.05)
    a = Engine.from_dir(mdir, dtype=dtype, kv_page_size=8, kv_cache_tokens=128, max_active_requests=2)
    b = Engine.from_config(cfg, seed=77, std=0.05, dtype=dtype, kv_page_size=8, kv_cache_tokens=128, max_active_requests=2)
    for la, lb in zip(a.model.layers, b.model.layers):
        assert torch.equal(la.mixer.w_qkv, lb.mixer.w_qkv) and torch.equal(la.mixer.b_qkv, lb.mixer.b_qkv)
        assert torch.equal(la.norm_mixer.weight, lb.norm_mixer.weight)
    assert torch.equal(a.model.embedding.table, b.model.embedding.table)
    toks = h.random_tokens(cfg, 50, seed=2)
    la = a.step([StepEntry("x", toks, list(range(50)))])
    lb = b.step([StepEntry("x", toks, list(range(50)))])
    assert torch.equal(la, lb)


def test_a_checkpoint_with_fused_experts_gives_the_same_logits(tmp_path, model_dirs):
    """The routed experts stored fused and input-major (``experts.gate_up_proj`` [E, H, 2I],
    ``experts.down_proj`` [E, I, H]) are cut and transposed at load: same logits as the converted layout."""
    import json
    import os

    from hi_b200.engine.core import Engine, StepEntry
    from hi_b200.weights import write_safetensors

    cfg, mdir = model_dirs["B"]
    w = h.read_weights(mdir)
    fused = {}
    for n, t in w.items():
        if n.endswith("experts.gate_proj.weight"):
            fused[n.replace("gate_proj.weight", "gate_up_proj")] = \
                torch.cat([t, w[n.replace("gate_proj", "up_proj")]], dim=1).transpose(1, 2).contiguous()
        elif n.endswith("experts.down_proj.weight"):
            fused[n[: -len(".weight")]] = t.transpose(1, 2).contiguous()
        elif not n.endswith("experts.up_proj.weight"):
            fused["language_model." + n] = t                   # and the prefix of a multimodal checkpoint
    out = tmp_path / "fused"
    os.makedirs(out)
    write_safetensors(str(out / "model.safetensors"), {("language_model." + n if not n.startswith("language_model.") else n): t
                                                        for n, t in fused.items()})
    json.dump(cfg, open(out / "config.json", "w"))
    toks = h.random_tokens(cfg, 40, seed=8)
    logits = [Engine.from_dir(d, dtype="float32", kv_page_size=16, kv_cache_tokens=64, max_active_requests=1)
              .step([StepEntry("x", toks, list(range(40)))]) for d in (mdir, str(out))]
    assert torch.equal(logits[0], logits[1])


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_the_float32_engine_against_the_cpu_reference(name, model_dirs):
    """The engine's float32 path (CUDA kernels, paged cache, portions) against the product tree's own
    CPU reference (plain C++ loops, whole sequence): within 1e-4 of the largest |logit|."""
    from hi_b200.engine.cpu_reference import CpuReference

    cfg, mdir = model_dirs[name]
    toks = h.random_tokens(cfg, 110, seed=33)
    want = CpuReference.from_dir(mdir).forward(toks)
    eng = engine_for(mdir, "float32", 8)
    got, _ = h.replay_in_process(eng, h.trace_portions({"x": toks}))
    out = torch.tensor(np.stack([got["x"][p] for p in range(len(toks))]))
    assert h.rel_err(out, want) <= 1e-4


def test_default_cache_size_comes_from_the_memory_that_is_free(model_dirs):
    """Without kv_cache_tokens the pools are sized from free device memory, capped at what the live
    requests can ever hold (max_position_embeddings each); generation runs in them."""
    import hi_b200

    cfg, mdir = model_dirs["A"]
    llm = hi_b200.LLM(mdir, dtype="float32", max_batch_size=2)
    groups = llm.engine.manager.snapshot()["groups"]
    keep = [g for g in groups if not g["window"]][0]
    chunked = [g for g in groups if g["window"]][0]
    assert keep["total"] * 64 == 2 * cfg["max_position_embeddings"]
    assert chunked["total"] * 64 <= 2 * cfg["max_position_embeddings"] and chunked["total"] >= 4
    outs = llm.generate([h.random_tokens(cfg, 20, seed=1)], hi_b200.SamplingParams(max_tokens=4, ignore_eos=True))
    assert outs[0].completion_tokens == 4


# --------------------------------------------------------------------------- a toy mixer with state
def test_toy_mixer_with_state_registers_builds_and_steps(model_dirs):
    """A mixer defined here, with per-request state of fixed size (a running mean of a projection),
    is registered, built into a model and stepped, without touching the framework's files."""
    from hi_b200.engine.core import Engine, StepEntry
    from hi_b200.parts import registry
    from hi_b200.parts.basic import Part
    from hi_b200.parts.model import Model
    from hi_b200.parts.spec import CacheSpec, LayerSpec, ModelSpec, PartSpec, TensorSpec
    from hi_b200.weights.loader import load_random

    @registry.register("mixer", "toy_running_mean")
    class ToyRunningMean(Part):
        def __init__(self, params, prefix, env):
            super().__init__(params, prefix, env)
            self.h, self.d = int(params["hidden_size"]), int(params["state_size"])

        def cache_spec(self):
            return CacheSpec(state_shape=(self.d + 1,))          # running sum and count

        def tensor_specs(self):
            return [TensorSpec(f"{self.prefix}.in.weight", (self.d, self.h)),
                    TensorSpec(f"{self.prefix}.out.weight", (self.h, self.d))]

        def load(self, fetch):
            self.w_in, self.w_out = fetch(f"{self.prefix}.in.weight"), fetch(f"{self.prefix}.out.weight")

        def forward(self, normed, ctx, cache):
            u = normed.float() @ self.w_in.float().T
            out = torch.empty_like(u)
            cu = [0]
            for n in ctx.n_new:
                cu.append(cu[-1] + n)
            for s, slot in enumerate(ctx.slot_ids):
                st = cache.state[slot]
                seg = u[cu[s]:cu[s + 1]]
                sums = st[: self.d] + torch.cumsum(seg, 0)
                counts = st[self.d] + torch.arange(1, seg.shape[0] + 1, device=u.device)
                out[cu[s]:cu[s + 1]] = sums / counts[:, None]
                st[: self.d], st[self.d] = sums[-1], counts[-1]
            return (out @ self.w_out.float().T).to(normed.dtype)

    try:
        H, V = 64, 97
        norm = lambda n: PartSpec("rmsnorm", {"name": n, "size": H, "eps": 1e-5})
        layers = []
        for i in range(3):
            mixer = PartSpec("toy_running_mean", {"name": "mix", "hidden_size": H, "state_size": 24}) if i != 1 else \
                PartSpec("attention", {"name": "attn", "hidden_size": H, "num_heads": 4, "num_kv_heads": 2, "head_dim": 16,
                                       "window": ("sliding", 9)})
            layers.append(LayerSpec(prefix=f"toy.layers.{i}", mixer=mixer, norm_mixer=norm("n1"), norm_feed_forward=norm("n2"),
                                    feed_forward=PartSpec("dense_swiglu", {"name": "ff", "hidden_size": H, "intermediate_size": 80})))
        spec = ModelSpec(hidden_size=H, vocab_size=V, layers=tuple(layers), schedule=ModelSpec.sequential(3),
                         embedding=PartSpec("token_embedding", {"name": "toy.embed", "vocab_size": V, "hidden_size": H}),
                         final_norm=norm("toy.norm"), head=PartSpec("linear_head", {"name": "toy.head", "vocab_size": V,
                                                                                    "hidden_size": H}))
        model = Model(spec, torch.float32, "cuda:0")
        load_random(model, seed=4, std=0.2)
        eng = Engine(model, kv_page_size=4, kv_cache_tokens=64, max_active_requests=3)
        assert [g.window for g in eng.manager.groups] == [("sliding", 9)]
        toks = {r: [(7 * i + 3 * k) % V for i in range(n)] for k, (r, n) in enumerate((("a", 40), ("b", 23)))}
        whole = {r: eng.step([StepEntry(r, t, list(range(len(t))))]) for r, t in toks.items()}
        for r in toks:
            eng.finish(r)
        # the same requests in portions, interleaved: state and window must carry over
        outs = {r: [] for r in toks}
        pos = {r: 0 for r in toks}
        sizes = [5, 1, 2, 7, 1, 3]
        i = 0
        while any(pos[r] < len(toks[r]) for r in toks):
            entries = []
            for r in toks:
                if pos[r] < len(toks[r]):
                    n = min(sizes[i % len(sizes)], len(toks[r]) - pos[r]); i += 1
                    entries.append(StepEntry(r, toks[r][pos[r]:pos[r] + n], list(range(n))))
                    pos[r] += n
            lg = eng.step(entries)
            row = 0
            for e in entries:
                outs[e.request_id].append(lg[row:row + len(e.tokens)]); row += len(e.tokens)
            eng.manager.check_invariants()
        for r in toks:
            got = torch.cat(outs[r])
            assert h.rel_err(got, whole[r].cpu()) <= 1e-4, f"toy mixer: request {r} differs between cuttings"
            eng.finish(r)
        sliding = eng.manager.snapshot()["groups"][0]
        assert sliding["peak"] <= 2 * (9 // 4 + 3), "the sliding window kept pages it had passed"
    finally:
        registry.unregister("mixer", "toy_running_mean")


# --------------------------------------------------------------------------- a toy position encoding and a toy routed feed-forward
def test_toy_position_and_toy_routed_feed_forward_against_a_plain_model():
    """A position encoding that is no rotation (a decay gamma^(query - key) put on q and k) and a
    feed-forward that routes each token to one of three tiny experts, both defined here, are
    registered, built into a model beside the framework's own parts, and stepped whole, in
    portions and token by token; the logits are compared with a plain model written out below
    from the plain functions and the toy formulas."""
    from hi_b200.engine.core import Engine, StepEntry
    from hi_b200.parts import registry
    from hi_b200.parts.basic import Part
    from hi_b200.parts.model import Model
    from hi_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, TensorSpec

    GAMMA = 0.97

    @registry.register("position", "toy_decay")
    class ToyDecay(Part):
        graph_safe = True

        def rotary_table(self):
            return None

        def apply(self, q, k, positions):
            decay = torch.exp(positions.to(torch.float32)[:, None, None] * math.log(GAMMA))   # device work only:
            return q.float() * decay, k.float() / decay                                          # the step may be captured

    @registry.register("feed_forward", "toy_three_experts")
    class ToyThreeExperts(Part):
        graph_safe = True

        def __init__(self, params, prefix, env):
            super().__init__(params, prefix, env)
            self.h = int(params["hidden_size"])

        def tensor_specs(self):
            return [TensorSpec(f"{self.prefix}.gate.weight", (3, self.h)),
                    TensorSpec(f"{self.prefix}.experts.weight", (3, self.h, self.h))]

        def load(self, fetch):
            self.gate, self.experts = fetch(f"{self.prefix}.gate.weight"), fetch(f"{self.prefix}.experts.weight")

        def forward(self, normed, ctx):
            x = normed.float()
            choice = (x @ self.gate.float().T).argmax(dim=1)
            w = self.experts.float()[choice]                          # [n, h, h]
            return torch.tanh(torch.einsum("nh,noh->no", x, w)).to(normed.dtype)

    try:
        H, V, NH, NKV, HD, EPS = 48, 61, 4, 2, 16, 1e-5
        norm = lambda n: PartSpec("rmsnorm", {"name": n, "size": H, "eps": EPS})
        attn = lambda pos, window: PartSpec("attention", {"name": "attn", "hidden_size": H, "num_heads": NH, "num_kv_heads": NKV,
                                                          "head_dim": HD, "window": window, "position": pos})
        rotary = PartSpec("rope", {"head_dim": HD, "theta": 10000.0, "scaling": None})
        layers = (
            LayerSpec(prefix="toy.layers.0", mixer=attn(PartSpec("toy_decay", {}), None), norm_mixer=norm("n1"),
                      norm_feed_forward=norm("n2"),
                      feed_forward=PartSpec("toy_three_experts", {"name": "ff", "hidden_size": H})),
            LayerSpec(prefix="toy.layers.1", mixer=attn(rotary, ("chunk", 12)), norm_mixer=norm("n1"), norm_feed_forward=norm("n2"),
                      feed_forward=PartSpec("dense_swiglu", {"name": "ff", "hidden_size": H, "intermediate_size": 56})),
        )
        spec = ModelSpec(hidden_size=H, vocab_size=V, layers=layers, schedule=ModelSpec.sequential(2),
                         embedding=PartSpec("token_embedding", {"name": "toy.embed", "vocab_size": V, "hidden_size": H}),
                         final_norm=norm("toy.norm"),
                         head=PartSpec("linear_head", {"name": "toy.head", "vocab_size": V, "hidden_size": H}))
        model = Model(spec, torch.float32, "cuda:0")
        g = torch.Generator().manual_seed(11)
        w = {}
        for ts in model.tensor_specs():
            if ts.init != "absent":                     # optional tensors (projection biases) stay out
                w[ts.name] = torch.ones(ts.shape) if ts.init == "ones" else torch.randn(ts.shape, generator=g) * 0.25
        model.load(lambda name: w[name].to("cuda:0") if name in w else None)
        eng = Engine(model, kv_page_size=4, kv_cache_tokens=96, max_active_requests=2)
        assert sorted(str(gr.window) for gr in eng.manager.groups) == ["('chunk', 12)", "None"]

        def plain_model(tokens):
            T = len(tokens)
            pos = torch.arange(T)
            x = w["toy.embed.weight"][tokens].float()
            inv = plain.rope_inverse_frequencies(HD, 10000.0, None)
            for i in range(2):
                p = f"toy.layers.{i}"
                z = plain.rms_norm(x, w[f"{p}.n1.weight"], EPS)
                q = (z @ w[f"{p}.attn.q_proj.weight"].T).reshape(T, NH, HD)
                k = (z @ w[f"{p}.attn.k_proj.weight"].T).reshape(T, NKV, HD)
                v = (z @ w[f"{p}.attn.v_proj.weight"].T).reshape(T, NKV, HD)
                if i == 0:      # the toy decay: score(t, s) = gamma^(t - s) q_t . k_s / sqrt(hd)
                    q, k = q * GAMMA ** pos[:, None, None], k * GAMMA ** (-pos[:, None, None].float())
                    a = plain.attention_core(q, k, v, None)
                else:
                    q, k = plain.apply_rope(q, pos, inv, False), plain.apply_rope(k, pos, inv, False)
                    a = plain.attention_core(q, k, v, 12)
                x = x + a @ w[f"{p}.attn.o_proj.weight"].T
                z = plain.rms_norm(x, w[f"{p}.n2.weight"], EPS)
                if i == 0:      # the toy experts: the largest gate logit picks one of three tanh layers
                    choice = (z @ w[f"{p}.ff.gate.weight"].T).argmax(dim=1)
                    x = x + torch.tanh(torch.einsum("nh,noh->no", z, w[f"{p}.ff.experts.weight"][choice]))
                else:
                    x = x + plain.swiglu(z, w[f"{p}.ff.gate_proj.weight"], w[f"{p}.ff.up_proj.weight"], w[f"{p}.ff.down_proj.weight"])
            return plain.rms_norm(x, w["toy.norm.weight"], EPS) @ w["toy.head.weight"].T

        toks = {"a": [(5 * i + 2) % V for i in range(41)], "b": [(11 * i + 7) % V for i in range(29)]}
        want = {r: plain_model(t) for r, t in toks.items()}
        for r, t in toks.items():                                   # whole
            got = eng.step([StepEntry(r, t, list(range(len(t))))]).cpu()
            eng.finish(r)
            assert h.rel_err(got, want[r]) <= 2e-5, f"toy parts, whole: request {r}"
        outs, at = {r: [] for r in toks}, {r: 0 for r in toks}      # both at once: portions, then token by token
        sizes, i = [6, 2, 9, 1, 4], 0
        while any(at[r] < len(toks[r]) for r in toks):
            entries = []
            for r, t in toks.items():
                if at[r] < len(t):
                    n = 1 if at[r] >= 24 else min(sizes[i % len(sizes)], len(t) - at[r]); i += 1
                    entries.append(StepEntry(r, t[at[r]:at[r] + n], list(range(n))))
                    at[r] += n
            lg, row = eng.step(entries).cpu(), 0
            for e in entries:
                outs[e.request_id].append(lg[row:row + len(e.tokens)]); row += len(e.tokens)
            eng.manager.check_invariants()
        for r in toks:
            assert h.rel_err(torch.cat(outs[r]), want[r]) <= 2e-5, f"toy parts, portions and decoding: request {r}"
            eng.finish(r)
    finally:
        registry.unregister("position", "toy_decay")
        registry.unregister("feed_forward", "toy_three_experts")


def test_the_tensor_core_kernels_take_the_sizes_they_are_built_for(tmp_path):
    """A silent fall to the general kernels would still give right logits: at head_dim 128 with
    64-token pages, a 300-token prompt and decoded tokens must go through the tcgen05 prefill
    attention, the fused TMA decode attention, the tcgen05 expert products (prompt) and the
    weight-streaming expert kernel (decode) in bfloat16, and through the general kernels in float32."""
    from hi_b200.engine.core import Engine, StepEntry
    from hi_b200.kernels import ops

    cfg = dict(TINY_A, hidden_size=256, num_attention_heads=8, num_key_value_heads=2, head_dim=128,
               attention_chunk_size=128, intermediate_size=128, intermediate_size_mlp=256, vocab_size=300)
    mdir = h.make_model(str(tmp_path / "m"), cfg, seed=3, std=0.04)
    toks = h.random_tokens(cfg, 310, seed=4)
    want = {"bfloat16": {"attention_prefill_tc", "attention_decode_fused", "moe_gate_up_tc", "moe_down_tc", "moe_gate_up",
                         "router_plan", "qkv_post", "add_rmsnorm"},
            "float32": {"paged_attention", "moe_gate_up", "moe_down", "router_plan"}}
    for dtype, tol in DTYPES:
        eng = Engine.from_dir(mdir, dtype=dtype, kv_page_size=64, kv_cache_tokens=512, max_active_requests=2)
        before = dict(ops.CALLS)
        steps = [([("a", toks[:300], list(range(300)))], [])] + [([("a", [toks[p]], [0])], []) for p in range(300, 310)]
        steps[-1] = (steps[-1][0], ["a"])
        got, forced = h.replay_in_process(eng, steps, record_routing=(dtype == "bfloat16"))
        ran = {k for k, v in ops.CALLS.items() if v > before.get(k, 0)}
        assert want[dtype] <= ran, f"{dtype}: {sorted(want[dtype] - ran)} did not run (ran: {sorted(ran)})"
        if dtype == "float32":
            assert not ran & {"attention_prefill_tc", "attention_decode_tma", "attention_decode_fused", "moe_gate_up_tc"}, "reduced-precision kernels on the 32-bit path"
        # and what they returned: every row against the plain model (bfloat16 given its own expert choices)
        h.compare_with_plain(cfg, h.read_weights(mdir), {"a": toks}, got, tol, forced=forced if dtype == "bfloat16" else None,
                             what=f"sizes of the fast kernels, {dtype}", margin=h.ROUTING_MARGIN)


def test_portions_far_into_a_context_share_their_keys_among_blocks(tmp_path, monkeypatch):
    """A short portion behind a long context gives the tensor-core prefill attention few blocks
    with long runs of keys; the global layers then let several blocks share a block's keys and a
    merge kernel combines their rows. The thresholds are lowered so that a 700-token request shows
    it (in use they ask for 32,768 cached tokens): portions of 130 and 140 tokens behind 384 and
    514, two requests side by side and a third that decodes beside them, every row against the plain model."""
    from hi_b200.engine.core import Engine
    from hi_b200.kernels import ops

    monkeypatch.setattr(ops, "PREFILL_SPLIT_MIN_TILES", 4)
    monkeypatch.setattr(ops, "PREFILL_SPLIT_MIN_SHARE", 1)
    cfg = dict(TINY_A, hidden_size=128, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
               attention_chunk_size=256, intermediate_size=64, intermediate_size_mlp=128, vocab_size=211,
               num_hidden_layers=4, nope_layer_interval=2)
    mdir = h.make_model(str(tmp_path / "m"), cfg, seed=9, std=0.05)
    # "c" decodes single tokens beside the portions of "a" and "b": its rows go through the decode kernel
    reqs = {"a": h.random_tokens(cfg, 700, seed=1), "b": h.random_tokens(cfg, 660, seed=2), "c": h.random_tokens(cfg, 43, seed=3)}
    cuts = {"a": [384, 130, 140, 46], "b": [400, 131, 129], "c": [40, 1, 1, 1]}
    steps, at = [], {r: 0 for r in reqs}
    for i in range(4):
        entries = []
        for r, sizes in cuts.items():
            if i < len(sizes):
                n = sizes[i]
                entries.append((r, reqs[r][at[r]: at[r] + n], list(range(n))))
                at[r] += n
        steps.append((entries, [r for r in reqs if at[r] == len(reqs[r]) and any(e[0] == r for e in entries)]))
    assert all(at[r] == len(reqs[r]) for r in reqs)
    seen = []
    real = ops.prefill_attention_tc

    def spy(*args, **kw):
        seen.append(kw.get("key_splits", 1))
        return real(*args, **kw)

    monkeypatch.setattr(ops, "prefill_attention_tc", spy)
    eng = Engine.from_dir(mdir, dtype="bfloat16", kv_page_size=16, kv_cache_tokens=1536, max_active_requests=3)
    got, forced = h.replay_in_process(eng, steps, record_routing=True)
    assert max(seen) > 1, f"no launch shared its keys (shares seen: {sorted(set(seen))})"
    assert 1 in seen, "the layers with chunked attention keep one block per query tile and head"
    h.compare_with_plain(cfg, h.read_weights(mdir), reqs, got, h.TOL_BF16, forced=forced,
                         what="keys shared among blocks", margin=h.ROUTING_MARGIN)

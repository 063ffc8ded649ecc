#!/usr/bin/env python3
"""Decode and prefill throughput of the Llama 4 engine on one B200, with roofline fractions.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--model scout|maverick] [--layers L]
                    [--batch B] [--context C] [--skip-extra]
    python bench.py --case NAME [sizes ...]        # one kernel or one step alone, for ncu

Default: the Scout-layer-sized 16-layer model with seeded random bfloat16 weights, batch 8,
8,192-token contexts. Token ids are uniform over the vocabulary; the caches of the decode
measurements are filled with seeded noise instead of being produced by a prefill (the bytes a
decode step reads are the same). One JSON line is printed:
  value            decoded tokens per second at the default batch, timed on the device
  e2e              the same through hi_b200.LLM (scheduler, sampler, host tokens in and out)
  prefill          one 2,048-token prompt in one step; frac = flops / time / bf16 peak
  roofline         bytes a decode step must read (every weight it uses once + live cache) / time
  points           decode tokens per second at batch 1 and 64, and the two further workloads:
  long_context     the same model at 65,536-token contexts: decoding at batch 1 and 4, and a prompt
                   fed in 4,096-token portions in the same steps as three decoding requests
                   (tokens per second of each portion against its offset, pages in use of the
                   chunked layers step by step: they fall back whenever the prompt passes 8,192)
  maverick         the 4-layer Maverick-sized model (128 experts), batch 64 at 4,096-token contexts:
                   tokens per second, roofline fraction, rows per expert of one step
  cpu_baseline_s   wall time of the plain implementation (tests/plain_llama4.py, whole sequences, no
                   cache, float32 on the CPU) on the two tiny workloads: the timed CPU baseline
The reference (PipeNetwork/hi) runs Llama 4 only through Apple MLX/Metal, so ``--impl
reference`` reports that it is unavailable here.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SCOUT = {
    "architectures": ["Llama4ForCausalLM"], "model_type": "llama4_text",
    "vocab_size": 202048, "hidden_size": 5120, "num_hidden_layers": 16,
    "num_attention_heads": 40, "num_key_value_heads": 8, "head_dim": 128, "rms_norm_eps": 1e-5,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 16.0, "low_freq_factor": 1.0, "high_freq_factor": 1.0,
                     "original_max_position_embeddings": 8192},
    "attention_chunk_size": 8192, "nope_layer_interval": 4, "use_qk_norm": True,
    "attn_temperature_tuning": True, "floor_scale": 8192, "attn_scale": 0.1,
    "interleave_moe_layer_step": 1, "num_local_experts": 16, "num_experts_per_tok": 1,
    "intermediate_size": 8192, "intermediate_size_mlp": 16384, "tie_word_embeddings": False,
    "max_position_embeddings": 262144,
}
MAVERICK = dict(SCOUT, num_hidden_layers=4, rope_scaling=None, use_qk_norm=False, interleave_moe_layer_step=2,
                num_local_experts=128)
MODELS = {"scout": (SCOUT, 16), "maverick": (MAVERICK, 4)}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
PAGE = 64
DEFAULT_STEPS = 64


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                p = json.load(f)
            return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p.get("bf16_tflops_sustained") or p["bf16_tflops"]),
                    "source": "measured"}
        except (ValueError, KeyError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """SM clock and throttle reasons during the timed regions (read-only NVML queries)."""

    def __init__(self):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(0)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
                 "hw_power_brake_slowdown": 0x80, "sync_boost": 0x10, "applications_clocks_setting": 0x2}
        while not self._stop.wait(0.2):
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                self.reasons |= {n for n, bit in names.items() if mask & bit}
            except Exception:
                pass

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons)}


def model_bytes_and_flops(model, distinct_by_layer, context):
    """From the built model: bytes of weights and cache one decode step must read for ONE request
    at ``context`` tokens (weights counted once, experts by how many distinct ones the step
    touched), the cache bytes per request, and the matrix flops per token."""
    weight_bytes, kv_bytes, flops = 0, 0, 0
    for i, layer in enumerate(model.layers):
        mix, ff = layer.mixer, layer.feed_forward
        attn = mix.w_qkv.numel() + mix.w_o.numel()
        weight_bytes += 2 * attn + 2 * 2 * model.spec.hidden_size
        flops += 2 * attn
        visible = context
        if mix.window:
            visible = ((context - 1) % mix.window[1]) + 1 if mix.window[0] == "chunk" else min(context, mix.window[1])
        kv_bytes += 2 * 2 * mix.nkv * mix.hd * visible
        if hasattr(ff, "w_gate"):
            expert = 3 * ff.hidden * ff.inter
            shared = ff.shared.w_gate_up.numel() + ff.shared.w_down.numel() if ff.shared else 0
            weight_bytes += 2 * (ff.w_router.numel() + shared + distinct_by_layer.get(i, ff.experts) * expert)
            flops += 2 * (ff.w_router.numel() + shared + ff.top_k * expert)
        else:
            dense = ff.mlp.w_gate_up.numel() + ff.mlp.w_down.numel()
            weight_bytes += 2 * dense
            flops += 2 * dense
    head = 2 * model.spec.vocab_size * model.spec.hidden_size
    return weight_bytes + head, kv_bytes, flops


def attention_flops(model, first, count):
    """Score and value flops of ``count`` new tokens at positions ``first ..`` (each query against
    the keys it may read: all earlier ones, or those of its own chunk)."""
    total = 0
    for layer in model.layers:
        mix = layer.mixer
        if mix.window and mix.window[0] == "chunk":
            c, keys, p, end = mix.window[1], 0, first, first + count
            while p < end:                               # chunk by chunk: a query at p sees p % c + 1 keys
                seg = min(end, (p // c + 1) * c) - p
                keys += seg * (p % c) + seg * (seg + 1) // 2
                p += seg
        else:
            keys = count * first + count * (count + 1) // 2
        total += 4 * mix.nh * mix.hd * keys
    return total


def build_engine(cfg, global_tokens, chunked_tokens, slots):
    """The model with random weights made on the device, pools of the given sizes (tokens), and
    caches filled with seeded noise (decode steps are timed without the prefill that would fill them)."""
    import torch

    from hi_b200.engine.core import Engine

    t0 = time.time()
    engine = Engine.from_config(cfg, seed=0, std=0.02, dtype="bfloat16", kv_page_size=PAGE,
                                kv_cache_tokens=global_tokens, windowed_cache_tokens=chunked_tokens,
                                max_active_requests=slots)
    torch.cuda.synchronize()
    load_s = time.time() - t0
    gen = torch.Generator(device="cuda").manual_seed(1)
    for view in engine.cache.views.values():
        if view.k_pages is not None:
            view.k_pages.normal_(0.0, 1.0, generator=gen)
            view.v_pages.normal_(0.0, 1.0, generator=gen)
    return engine, load_s


def timed_decode(engine, batch, ctx_len, steps, warmup, vocab, cpu_gen, tag="d"):
    """W + K single-token steps of ``batch`` requests whose contexts end at ``ctx_len``; the K
    timed steps lie between two synchronisations, every step has its own event too (median)."""
    import torch

    from hi_b200.engine.core import StepEntry
    from hi_b200.kernels import ops

    total = warmup + steps + 1
    ids = [f"{tag}{batch}-{i}" for i in range(batch)]
    for rid in ids:
        engine.assume_cached(rid, ctx_len - total)
    toks = torch.randint(0, vocab, (total, batch), generator=cpu_gen).tolist()
    # one step with a tap to see which experts a step touches, then the warm-up steps (the first
    # step of a shape is eager, the second captures the CUDA graph of this shape)
    taps = {}
    engine.step([StepEntry(r, [toks[total - 1][i]], [0]) for i, r in enumerate(ids)],
                tap=lambda n, t: taps.__setitem__(n, t.clone()))
    routing = {int(n.split(".")[2]): t.flatten().tolist() for n, t in taps.items() if n.endswith("router_ids")}
    distinct = {layer: len(set(chosen)) for layer, chosen in routing.items()}
    for s in range(warmup):
        engine.step([StepEntry(r, [toks[s][i]], [0]) for i, r in enumerate(ids)])
    torch.cuda.synchronize()
    launches0 = ops.LAUNCHES[0]
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    marks[0].record()
    for k, s in enumerate(range(warmup, total - 1)):
        engine.step([StepEntry(r, [toks[s][i]], [0]) for i, r in enumerate(ids)])
        marks[k + 1].record()
    torch.cuda.synchronize()
    ms = marks[0].elapsed_time(marks[-1]) / steps
    per_step = [marks[k].elapsed_time(marks[k + 1]) for k in range(steps)]
    launches = ops.LAUNCHES[0] - launches0
    for rid in ids:
        engine.finish(rid)
    wb, kv, _ = model_bytes_and_flops(engine.model, distinct, ctx_len)
    return {"ms": ms, "ms_median": statistics.median(per_step), "tok_s": batch * 1000.0 / ms, "launches": launches,
            "distinct": (sum(distinct.values()) / len(distinct) if distinct else 0.0), "bytes": wb + batch * kv,
            "routing": routing}


def release(engine):
    import torch

    engine.model = None
    engine.cache = None
    engine._graphs.clear()
    del engine
    gc.collect()
    torch.cuda.empty_cache()


def long_context_point(engine, cfg, args, pk, vocab, cpu_gen):
    """65,536-token contexts on the same model: decoding at batch 1 and 4, and one request's prompt
    fed in 4,096-token portions in the same steps as three requests that decode."""
    import torch

    from hi_b200.engine.core import StepEntry

    ctx = args.long_context
    out = {"context": ctx}
    steps = max(8, min(args.steps, 32))
    for b in (1, 4):
        r = timed_decode(engine, b, ctx, steps, args.warmup, vocab, cpu_gen, tag="L")
        out[f"decode_b{b}"] = {"value": r["tok_s"], "ms_per_step": r["ms"],
                               "frac": r["bytes"] / (r["ms"] * 1e-3) / 1e9 / pk["hbm_gbs"]}
    portion = args.long_portion
    n_portions = (ctx - portion) // portion
    decoders = [f"Lm{i}" for i in range(3)]
    for rid in decoders:
        engine.assume_cached(rid, ctx - n_portions - 4)
    prompt = torch.randint(0, vocab, (n_portions * portion,), generator=cpu_gen).tolist()
    dec = torch.randint(0, vocab, (n_portions + 1, 3), generator=cpu_gen).tolist()
    chunked = [g for g, spec in enumerate(engine.manager.groups) if spec.window]
    portions, pages = [], []
    # the first portion runs once untimed (warm-up of this step shape), as a request of its own
    engine.step([StepEntry("Lwarm", prompt[:portion], [])] + [StepEntry(r, [dec[n_portions][i]], [0]) for i, r in enumerate(decoders)])
    engine.finish("Lwarm")
    torch.cuda.synchronize()
    for p in range(n_portions):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        entries = [StepEntry("Lp", prompt[p * portion:(p + 1) * portion], [portion - 1] if p == n_portions - 1 else [])]
        entries += [StepEntry(r, [dec[p][i]], [0]) for i, r in enumerate(decoders)]
        start.record()
        engine.step(entries)
        end.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(end)
        _, _, fpt = model_bytes_and_flops(engine.model, {}, ctx)
        flops = fpt * (portion + 3) + attention_flops(engine.model, p * portion, portion)
        portions.append({"offset": p * portion, "ms": round(ms, 2), "tokens_per_s": round((portion + 3) * 1000.0 / ms),
                         "frac": round(flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 3)})
        snap = engine.manager.snapshot()["groups"]
        pages.append(sum(snap[g]["used"] for g in chunked))
    for rid in decoders + ["Lp"]:
        engine.finish(rid)
    out["mixed_steps"] = {"portion_tokens": portion, "decoding_requests": 3, "portions": portions,
                          "chunked_pages_in_use_after_each_step": pages, "page_tokens": PAGE}
    # a short portion far into a context: few blocks with long runs of keys, which the layers that
    # see every key share out among several blocks each; timed with that and without
    from hi_b200.kernels import ops

    short = 512
    engine.assume_cached("Ls", ctx - 4 * short)
    toks = torch.randint(0, vocab, (3 * short,), generator=cpu_gen).tolist()
    times = []
    for i, min_tiles in enumerate((None, None, 1 << 30)):       # the first runs untimed
        keep = ops.PREFILL_SPLIT_MIN_TILES
        if min_tiles:
            ops.PREFILL_SPLIT_MIN_TILES = min_tiles
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        engine.step([StepEntry("Ls", toks[i * short:(i + 1) * short], [])])
        end.record()
        torch.cuda.synchronize()
        ops.PREFILL_SPLIT_MIN_TILES = keep
        times.append(start.elapsed_time(end))
    engine.finish("Ls")
    out["short_portion"] = {"tokens": short, "offset": ctx - 3 * short, "ms": round(times[1], 2),
                            "ms_one_block_per_query_tile": round(times[2], 2)}
    return out


def maverick_point(args, pk, cpu_gen):
    """The Maverick-sized model (4 layers, two of them with 128 experts), batch 64, 4,096-token contexts."""
    cfg, _full = MODELS["maverick"]
    engine, load_s = build_engine(cfg, 64 * (4096 + PAGE) + 4 * PAGE, 64 * (4096 + 2 * PAGE) + 4 * PAGE, 66)
    r = timed_decode(engine, 64, 4096, max(8, min(args.steps, 32)), args.warmup, cfg["vocab_size"], cpu_gen, tag="M")
    rows = {}
    for layer, chosen in r["routing"].items():
        counts = {}
        for e in chosen:
            counts[e] = counts.get(e, 0) + 1
        hist = {}
        for c in counts.values():
            hist[c] = hist.get(c, 0) + 1
        rows[f"layer{layer}"] = {"experts_with_rows": len(counts), "max_rows": max(counts.values()),
                                 "mean_rows": round(len(chosen) / len(counts), 2),
                                 "experts_by_rows": {str(k): hist[k] for k in sorted(hist)}}
    out = {"value": r["tok_s"], "ms_per_step": r["ms"], "batch": 64, "context": 4096, "layers": cfg["num_hidden_layers"],
           "experts": cfg["num_local_experts"], "bytes_per_step": r["bytes"],
           "frac": r["bytes"] / (r["ms"] * 1e-3) / 1e9 / pk["hbm_gbs"], "rows_per_expert": rows,
           "weights_load_s": round(load_s, 1)}
    release(engine)
    return out


def cpu_baseline():
    """Wall time of the plain implementation on the two tiny workloads (4 prompts of 7/19/33/48 tokens
    + 16 generated tokens each on tiny A; 3 prompts of 5/40/70 + 24 on tiny B): greedy generation
    that runs the whole sequence again for every token, float32 on the CPU."""
    import tempfile

    import torch

    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import plain_llama4 as plain
    from harness import make_model, random_tokens, read_weights
    from tiny_configs import TINY_A, TINY_B

    out = {}
    threads = torch.get_num_threads()
    for name, cfg, prompts, new in (("tiny_a", TINY_A, (7, 19, 33, 48), 16), ("tiny_b", TINY_B, (5, 40, 70), 24)):
        with tempfile.TemporaryDirectory() as d:
            make_model(d, cfg, seed=11, std=0.08)
            w = read_weights(d)
        t0 = time.perf_counter()
        for i, n in enumerate(prompts):
            toks = random_tokens(cfg, n, seed=50 + i)
            for _ in range(new):
                toks.append(int(plain.forward(cfg, w, toks)[-1].argmax()))
        out[name] = round(time.perf_counter() - t0, 2)
    out["threads"] = threads
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=DEFAULT_STEPS)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="scout", choices=sorted(MODELS))
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--points", default="1,64")
    ap.add_argument("--skip-prefill", action="store_true")
    ap.add_argument("--skip-extra", action="store_true", help="leave out the long-context, Maverick and CPU points")
    ap.add_argument("--long-context", type=int, default=65536)
    ap.add_argument("--long-portion", type=int, default=4096)
    ap.add_argument("--case", nargs="+", default=None, metavar=("NAME", "SIZE"),
                    help="run one kernel or one step alone a few times (for ncu): " + ", ".join(sorted(CASES)))
    args = ap.parse_args(argv)
    if args.case:
        CASES[args.case[0]](*[int(a) for a in args.case[1:]])
        print("ok")
        return 0
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "PipeNetwork/hi runs Llama 4 only through Apple MLX/Metal (crates/hi-mlx, macOS aarch64); "
                          "it is a Rust workspace with no Python package and no Rust toolchain is installed here"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is outside this engine (single-GPU by design)")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch

    import hi_b200
    from hi_b200.engine.core import StepEntry
    from hi_b200.sampling import SamplingParams

    pk = peaks()
    base_cfg, FULL_LAYERS = MODELS[args.model]
    if args.layers is None:
        args.layers = FULL_LAYERS
    cfg = dict(base_cfg, num_hidden_layers=args.layers)
    points = sorted({int(p) for p in args.points.split(",") if p} | {args.batch})
    max_batch = max(points)
    ctx_len = args.context
    extra = not args.skip_extra and args.model == "scout" and args.layers == FULL_LAYERS
    # pools: every request of the largest batch at the context length, the prompt of the prefill point and
    # some slack; rotary layers keep one attention chunk per request (plus the pages being written).
    # The long-context point reuses this engine: four requests of 65,536 tokens, one of them fed in portions
    slack = args.prefill_tokens + 4 * PAGE
    global_tokens = max_batch * (ctx_len + PAGE) + slack
    chunked_tokens = max_batch * (min(ctx_len, cfg["attention_chunk_size"]) + 2 * PAGE) + slack
    if extra:
        global_tokens = max(global_tokens, 4 * (args.long_context + PAGE) + slack)
        chunked_tokens = max(chunked_tokens, 4 * (cfg["attention_chunk_size"] + 2 * PAGE) + args.long_portion + slack)
    engine, load_s = build_engine(cfg, global_tokens, chunked_tokens, max(max_batch, 4) + 2)
    vocab = cfg["vocab_size"]
    cpu_gen = torch.Generator().manual_seed(2)
    sampler = ClockSampler()
    sampler.start()

    results = {b: timed_decode(engine, b, ctx_len, args.steps, args.warmup, vocab, cpu_gen) for b in points}
    main_r = results[args.batch]

    # ---- prefill: one prompt of --prefill-tokens in one step, logits at the last position
    prefill = None
    if not args.skip_prefill:
        T = args.prefill_tokens
        reps = 3
        times = []
        for r in range(reps + 1):
            toks = torch.randint(0, vocab, (T,), generator=cpu_gen).tolist()
            torch.cuda.synchronize()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            engine.step([StepEntry("p", toks, [T - 1])])
            end.record()
            torch.cuda.synchronize()
            engine.finish("p")
            if r > 0:
                times.append(start.elapsed_time(end))
        ms = statistics.median(times)
        _, _, fpt = model_bytes_and_flops(engine.model, {}, T)
        nh, hd = cfg["num_attention_heads"], cfg["head_dim"]
        flops = fpt * T + args.layers * 4 * nh * hd * T * T / 2 + 2 * vocab * cfg["hidden_size"]
        prefill = {"value": T * 1000.0 / ms, "tokens": T, "ms": ms, "frac": flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12),
                   "peak_tflops": pk["bf16_tflops"], "peak_source": pk["source"]}

    # ---- end to end through the public entry point: scheduler + sampler, host tokens in and out
    llm = hi_b200.LLM(engine, max_batch_size=args.batch, max_batched_tokens=8192)
    total = args.warmup + args.steps
    reqs = []
    for i in range(args.batch):
        prompt = torch.randint(0, vocab, (ctx_len - total,), generator=cpu_gen).tolist()
        req = llm.add_request(prompt, SamplingParams(max_tokens=total, ignore_eos=True, temperature=0.0), request_id=f"e{i}")
        reqs.append(req)
    # the prompts' keys are taken as cached noise except for their last token
    for req in reqs:
        engine.assume_cached(req.request_id, len(req.prompt) - 1)
        llm.scheduler.assume_running(req, len(req.prompt) - 1)
    for _ in range(args.warmup):
        llm.step()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall = time.perf_counter()
    start.record()
    n_steps = 0
    # tokens the host has read so far, and those of the step that is already running (launched by
    # the last warm-up call; its work lies before the timed region, so its tokens do not count)
    read_before = sum(len(r.output) for r in reqs) + (len(llm._launched.sampling) if llm._launched is not None else 0)
    while any(r.status != "finished" for r in reqs):
        llm.step()
        n_steps += 1
    end.record()
    torch.cuda.synchronize()
    wall_ms = (time.perf_counter() - t_wall) * 1000.0
    # tokens that reached the host inside the timed region (a step launched ahead is read one call later)
    e2e_tok_s = (sum(len(r.output) for r in reqs) - read_before) * 1000.0 / max(wall_ms, start.elapsed_time(end))
    h2d = engine.last_step_h2d_bytes          # the packed step inputs (tokens, positions, block tables, ...)
    clocks = sampler.stop()

    line = {
        "metric": f"decode tokens/s (Llama 4 {args.model.capitalize()} layer sizes, bf16)", "value": main_r["tok_s"], "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": main_r["ms"],
        "ms_per_step_median": main_r["ms_median"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights N(0,0.02), uniform random token ids, noise-filled KV cache",
        "config": {"model": f"llama4-{args.model}-layers", "layers": args.layers, "layers_full": FULL_LAYERS,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "experts": cfg["num_local_experts"], "top_k": cfg["num_experts_per_tok"],
                   "expert_inter": cfg["intermediate_size"], "mlp_inter": cfg["intermediate_size_mlp"],
                   "moe_every": cfg.get("interleave_moe_layer_step", 1), "vocab": vocab, "chunk": cfg["attention_chunk_size"],
                   "global_batch": args.batch, "seq_len": ctx_len, "page": PAGE, "parallelism": "single-gpu",
                   "l2": "inputs larger than L2 (each step streams all weights it uses)",
                   "weights_load_s": round(load_s, 1)},
        "clocks": clocks,
        "e2e": {"value": e2e_tok_s, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * args.batch,
                "steps": n_steps},
        "gpu_launches": main_r["launches"],
        "roofline": {"bound": "hbm", "achieved": main_r["bytes"] / (main_r["ms"] * 1e-3) / 1e9, "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": main_r["bytes"] / (main_r["ms"] * 1e-3) / 1e9 / pk["hbm_gbs"],
                     "peak_source": pk["source"], "bytes_per_step": main_r["bytes"],
                     "distinct_experts_per_layer": main_r["distinct"]},
        "points": {f"decode_b{b}": results[b]["tok_s"] for b in points if b != args.batch},
        "points_roofline_frac": {f"decode_b{b}": results[b]["bytes"] / (results[b]["ms"] * 1e-3) / 1e9 / pk["hbm_gbs"]
                                 for b in points},
    }
    if prefill:
        line["prefill"] = prefill
    if extra:
        long_ctx = long_context_point(engine, cfg, args, pk, vocab, cpu_gen)
        line["long_context"] = long_ctx
        line["points"]["decode_b1_ctx65536"] = long_ctx["decode_b1"]["value"]
        line["points"]["decode_b4_ctx65536"] = long_ctx["decode_b4"]["value"]
        llm = None
        release(engine)
        mav = maverick_point(args, pk, cpu_gen)
        line["maverick"] = mav
        line["points"]["maverick_decode_b64_ctx4096"] = mav["value"]
        line["cpu_baseline_s"] = cpu_baseline()
    print(json.dumps(line))
    return 0


# --------------------------------------------------------------------------- one kernel or one step alone
# Small, fixed cases at the Scout layer's sizes (40 heads, 8 kv heads, head_dim 128; hidden 5120,
# 16 experts of 8192) for `ncu -k regex:<kernel>`: inputs larger than L2, a few GB at most.
DEV = "cuda:0"


def case_decode_attention(batch=8, context=8192, page=64):
    import torch

    from hi_b200.kernels import ops

    nh, nkv, hd = 40, 8, 128
    blocks = -(-context // page)
    g = torch.Generator(device=DEV).manual_seed(0)
    kp = torch.randn(batch * blocks, nkv, page, hd, device=DEV, generator=g).to(torch.bfloat16)
    vp = torch.randn(batch * blocks, nkv, page, hd, device=DEV, generator=g).to(torch.bfloat16)
    bt = torch.randperm(batch * blocks, device=DEV, generator=g).to(torch.int32).view(batch, blocks).contiguous()
    q = torch.randn(batch, nh, hd, device=DEV, generator=g).to(torch.bfloat16)
    pos = torch.full((batch,), context - 1, dtype=torch.int32, device=DEV)
    sot = torch.arange(batch, dtype=torch.int32, device=DEV)
    for _ in range(3):
        ops.decode_attention(q, kp, vp, bt, sot, pos, 0, 0, hd ** -0.5, context)
    torch.cuda.synchronize()


def case_decode_attention_fused(batch=8, context=8192, page=64):
    """The one-launch form: q/k/v encoding, cache append, attention and merge, on a rotary chunked layer's settings."""
    import torch

    from hi_b200.kernels import ops

    nh, nkv, hd = 40, 8, 128
    blocks = -(-context // page)
    g = torch.Generator(device=DEV).manual_seed(0)
    kp = torch.randn(batch * blocks, nkv, page, hd, device=DEV, generator=g).to(torch.bfloat16)
    vp = torch.randn(batch * blocks, nkv, page, hd, device=DEV, generator=g).to(torch.bfloat16)
    bt = torch.randperm(batch * blocks, device=DEV, generator=g).to(torch.int32).view(batch, blocks).contiguous()
    qkv = torch.randn(batch, (nh + 2 * nkv) * hd, device=DEV, generator=g).to(torch.bfloat16)
    pos = torch.full((batch,), context - 1, dtype=torch.int32, device=DEV)
    sot = torch.arange(batch, dtype=torch.int32, device=DEV)
    inv = torch.rand(hd // 2, device=DEV, generator=g)
    for _ in range(3):
        ops.decode_attention_fused(qkv, nh, nkv, hd, pos, inv, False, True, 1e-6, None, sot, bt, kp, vp, 8192, 0, hd ** -0.5, context)
    torch.cuda.synchronize()


def _experts(experts, rows):
    import torch

    from hi_b200.kernels import ops

    hidden, inter = 5120, 8192
    g = torch.Generator(device=DEV).manual_seed(0)
    x = torch.randn(rows, hidden, device=DEV, generator=g).to(torch.bfloat16)
    wg = (torch.randn(experts, inter, hidden, device=DEV, generator=g) * 0.02).to(torch.bfloat16)
    wu = (torch.randn(experts, inter, hidden, device=DEV, generator=g) * 0.02).to(torch.bfloat16)
    wd = (torch.randn(experts, hidden, inter, device=DEV, generator=g) * 0.02).to(torch.bfloat16)
    ids = torch.randint(0, experts, (rows, 1), device=DEV, generator=g).to(torch.int32)
    scores = torch.rand(rows, 1, device=DEV, generator=g)
    return x, wg, wu, wd, scores, ops.moe_plan(ids, experts)


def case_expert_gemv(batch=8):
    """The weight-streaming expert kernels at decode shape."""
    import torch

    from hi_b200.kernels import ops

    x, wg, wu, wd, scores, plan = _experts(16, batch)
    for _ in range(3):
        act = ops.moe_gate_up(x, plan, 1, wg, wu, scores, True)
        ops.moe_down(act, wd, plan, True)
    torch.cuda.synchronize()


def case_expert_tc(tokens=1024, experts=8):
    """The tcgen05 grouped products at prefill shape: about 128 rows per expert."""
    from hi_b200.kernels import ops

    x, wg, wu, wd, scores, plan = _experts(experts, tokens)
    for _ in range(3):
        act = ops.moe_gate_up_tc(x, plan, 1, wg, wu, scores)
        ops.moe_down_tc(act, wd, plan)
    ops.check_tc_status()


def case_prefill_attention(tokens=2048, cached=0, page=64):
    """One portion of ``tokens`` new tokens behind ``cached`` earlier ones, both prefill kernels."""
    import torch

    from hi_b200.kernels import ops

    nh, nkv, hd = 40, 8, 128
    total = tokens + cached
    blocks = -(-total // page)
    g = torch.Generator(device=DEV).manual_seed(0)
    kp = torch.randn(blocks, nkv, page, hd, device=DEV, generator=g).to(torch.bfloat16)
    vp = torch.randn(blocks, nkv, page, hd, device=DEV, generator=g).to(torch.bfloat16)
    bt = torch.randperm(blocks, device=DEV, generator=g).to(torch.int32).view(1, blocks).contiguous()
    q = torch.randn(tokens, nh, hd, device=DEV, generator=g).to(torch.bfloat16)
    pos = torch.arange(cached, total, dtype=torch.int32, device=DEV)
    cu = torch.tensor([0, tokens], dtype=torch.int32, device=DEV)
    for _ in range(3):
        if cached == 0:
            ops.prefill_attention(q, kp, vp, bt, cu, pos, 1, tokens, 0, 0, hd ** -0.5)
        ops.prefill_attention_tc(q, kp, vp, bt, cu, pos, 1, tokens, 0, 0, hd ** -0.5)
    ops.check_tc_status()


def _case_engine(layers, tokens, slots):
    from hi_b200.engine.core import Engine

    return Engine.from_config(dict(SCOUT, num_hidden_layers=layers), seed=0, dtype="bfloat16", device=DEV,
                              kv_page_size=PAGE, kv_cache_tokens=tokens, max_active_requests=slots, use_cuda_graphs=False)


def case_decode_step(batch=8, context=8192, layers=2):
    """Three decode steps of ``batch`` requests at ``context`` cached tokens, every kernel launched on its own."""
    import torch

    from hi_b200.engine.core import StepEntry

    eng = _case_engine(layers, batch * (context + 128), batch + 1)
    for i in range(batch):
        eng.assume_cached(i, context - 8)
    g = torch.Generator().manual_seed(0)
    for _ in range(3):
        eng.step([StepEntry(i, [int(torch.randint(0, 202048, (1,), generator=g))], [0]) for i in range(batch)])
    torch.cuda.synchronize()


def case_prefill_step(tokens=2048, layers=2):
    """Three prompts of ``tokens`` tokens, each in one step."""
    import torch

    from hi_b200.engine.core import StepEntry

    eng = _case_engine(layers, tokens + 128, 2)
    g = torch.Generator().manual_seed(0)
    for i in range(3):
        eng.step([StepEntry(i, torch.randint(0, 202048, (tokens,), generator=g).tolist(), [tokens - 1])])
        eng.finish(i)
    torch.cuda.synchronize()


def case_sweep():
    """The hot kernels alone over further sizes, timed with CUDA events (median of five, a buffer
    larger than L2 written between calls), with their fractions of the measured peaks: decode
    attention by batch and context, the expert products by the number of routed tokens (the kernel
    the feed-forward part would pick), prefill attention by portion length and offset. Markdown."""
    import torch

    from hi_b200.kernels import ops
    from hi_b200.parts.attention import AttentionMixer
    from hi_b200.parts.feed_forward import SigmoidRoutedExperts

    pk = peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)
    g = torch.Generator(device=DEV).manual_seed(0)

    def timed(fn):
        fn()
        ts = []
        for _ in range(5):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1e3)
        return sorted(ts)[2]

    nh, nkv, hd, page = 40, 8, 128, 64
    print(f"peaks: {pk['hbm_gbs']:.1f} GB/s copy, {pk['bf16_tflops']:.1f} TFLOP/s bf16 ({pk['source']}); times include the launch\n")
    print("decode attention, 40 heads / 8 kv heads, head_dim 128 (one launch: q/k/v encoding, append, attention, merge; "
          "from 256 (token, kv head) pairs on: qkv_post + attention + merge)\n")
    print("| requests | keys each | us | GB/s of K and V | of the copy peak |\n|---|---|---|---|---|")
    for context in (1024, 8192, 32768, 65536):
        for batch in (1, 2, 4, 8, 16, 32, 64):
            if batch * context > 64 * 8192 * 2:
                continue
            blocks = -(-context // page)
            kp = torch.randn(batch * blocks, nkv, page, hd, device=DEV, generator=g).to(torch.bfloat16)
            vp = torch.randn(batch * blocks, nkv, page, hd, device=DEV, generator=g).to(torch.bfloat16)
            bt = torch.randperm(batch * blocks, device=DEV, generator=g).to(torch.int32).view(batch, blocks).contiguous()
            qkv = torch.randn(batch, (nh + 2 * nkv) * hd, device=DEV, generator=g).to(torch.bfloat16)
            pos = torch.full((batch,), context - 1, dtype=torch.int32, device=DEV)
            sot = torch.arange(batch, dtype=torch.int32, device=DEV)

            def attend():
                o = ops.decode_attention_fused(qkv, nh, nkv, hd, pos, None, False, True, 1e-6, (8192.0, 0.1), sot, bt, kp, vp,
                                               0, 0, hd ** -0.5, context)
                if o is None:
                    q = ops.qkv_post(qkv, nh, nkv, hd, pos, None, False, True, 1e-6, (8192.0, 0.1), sot, bt, kp, vp, page, True)
                    ops.decode_attention(q, kp, vp, bt, sot, pos, 0, 0, hd ** -0.5, context)

            us = timed(attend)
            gbs = batch * context * 2 * nkv * hd * 2 / us / 1e3
            print(f"| {batch} | {context} | {us:.1f} | {gbs:.0f} | {gbs / pk['hbm_gbs']:.2f} |")
            del kp, vp
    x, wg, wu, wd, scores, _plan = _experts(16, 4096)
    print("\nrouted experts, 16 experts top-1, hidden 5120, intermediate 8192: gate/up + SwiGLU, then down\n")
    print("| tokens | experts with rows | kernels | us | GB/s of expert weights | of the copy peak |\n|---|---|---|---|---|---|")
    for n in (1, 2, 4, 8, 10, 12, 16, 32, 64, 128, 256, 512, 1024, 2048, 4096):
        ids = torch.randint(0, 16, (n, 1), device=DEV, generator=g).to(torch.int32)
        plan = ops.moe_plan(ids, 16)
        distinct = int(torch.unique(ids).numel())
        few = n <= SigmoidRoutedExperts.FEW_ROWS

        def experts():
            if few:
                ops.moe_down(ops.moe_gate_up(x[:n], plan, 1, wg, wu, scores[:n], True), wd, plan, True)
            else:
                ops.moe_down_tc(ops.moe_gate_up_tc(x[:n], plan, 1, wg, wu, scores[:n]), wd, plan)

        us = timed(experts)
        gbs = distinct * 3 * 8192 * 5120 * 2 / us / 1e3
        print(f"| {n} | {distinct} | {'weight streaming' if few else 'tcgen05'} | {us:.1f} | {gbs:.0f} | {gbs / pk['hbm_gbs']:.2f} |")
    ops.check_tc_status()
    del x, wg, wu, wd
    print("\nprefill attention (tcgen05), one request, 40 heads / 8 kv heads, head_dim 128, a layer that sees every key\n")
    print("| new tokens | cached before | key shares | us | TFLOP/s | of sustained bf16 |\n|---|---|---|---|---|---|")
    for cached in (0, 8192, 61440):
        for tokens in (128, 256, 512, 1024, 2048, 4096, 8192):
            if cached and tokens > 4096:
                continue
            total = tokens + cached
            blocks = -(-total // page)
            kp = torch.randn(blocks, nkv, page, hd, device=DEV, generator=g).to(torch.bfloat16)
            vp = torch.randn(blocks, nkv, page, hd, device=DEV, generator=g).to(torch.bfloat16)
            bt = torch.randperm(blocks, device=DEV, generator=g).to(torch.int32).view(1, blocks).contiguous()
            q = torch.randn(tokens, nh, hd, device=DEV, generator=g).to(torch.bfloat16)
            pos = torch.arange(cached, total, dtype=torch.int32, device=DEV)
            cu = torch.tensor([0, tokens], dtype=torch.int32, device=DEV)
            shares = 1
            if cached >= 2 * tokens:
                shares = ops.prefill_key_splits(nh * -(-tokens // 128), cached // 64, ops.sm_count(DEV))
            us = timed(lambda: ops.prefill_attention_tc(q, kp, vp, bt, cu, pos, 1, tokens, 0, 0, hd ** -0.5, key_splits=shares))
            tf = 4 * nh * hd * (tokens * cached + tokens * (tokens + 1) / 2) / us / 1e6
            print(f"| {tokens} | {cached} | {shares} | {us:.1f} | {tf:.0f} | {tf / pk['bf16_tflops']:.2f} |")
            del kp, vp
    ops.check_tc_status()


def _timeline(run, warm, what):
    """Kernel starts and ends of one step from the profiler's activity records (real durations, with
    what runs beside what), as markdown: the first two layers' launches, then totals by kernel."""
    import torch
    from torch.profiler import ProfilerActivity, profile

    for _ in range(warm):
        run()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        run()
        torch.cuda.synchronize()
    evs = [e for e in prof.events() if e.device_type.name == "CUDA" and "emcpy" not in e.name and "emset" not in e.name]
    evs.sort(key=lambda e: e.time_range.start)
    name = lambda e: e.name.replace("void ", "").replace("(anonymous namespace)::", "").split("(")[0][:58]
    t0 = evs[0].time_range.start
    span = evs[-1].time_range.end - t0
    print(f"{what}: {len(evs)} kernels in {span:.0f} us\n")
    print("| start us | end us | us | kernel |\n|---|---|---|---|")
    norms = 0
    for e in evs:
        norms += "add_rmsnorm" in e.name
        if norms > 5:                       # two layers: four norms, then the third layer's first
            break
        print(f"| {e.time_range.start - t0:.1f} | {e.time_range.end - t0:.1f} | {e.time_range.end - e.time_range.start:.1f} | {name(e)} |")
    agg = {}
    for e in evs:
        a = agg.setdefault(name(e), [0, 0.0])
        a[0] += 1
        a[1] += e.time_range.end - e.time_range.start
    print("\n| kernel | launches | us in all | us each |\n|---|---|---|---|")
    for k, (c, v) in sorted(agg.items(), key=lambda kv: -kv[1][1]):
        print(f"| {k} | {c} | {v:.1f} | {v / c:.1f} |")


def case_decode_timeline(batch=8, context=8192, layers=4):
    """One captured decode step of ``batch`` requests at ``context`` cached tokens: when each kernel ran."""
    import torch

    from hi_b200.engine.core import StepEntry

    eng = _case_engine(layers, batch * (context + 128), batch + 1)
    eng.use_cuda_graphs = True
    for view in eng.cache.views.values():
        view.k_pages.normal_(); view.v_pages.normal_()
    for i in range(batch):
        eng.assume_cached(i, context - 16)
    g = torch.Generator().manual_seed(0)
    step = lambda: eng.step([StepEntry(i, [int(torch.randint(0, 202048, (1,), generator=g))], [0]) for i in range(batch)])
    _timeline(step, 6, f"decode step, {batch} requests x {context} cached tokens, {layers} Scout-sized layers, captured graph")


def case_prefill_timeline(tokens=2048, layers=4):
    """One prompt of ``tokens`` tokens in one step: when each kernel ran."""
    import torch

    from hi_b200.engine.core import StepEntry

    eng = _case_engine(layers, tokens + 128, 2)
    g = torch.Generator().manual_seed(0)
    count = [0]

    def step():
        count[0] += 1
        eng.step([StepEntry(count[0], torch.randint(0, 202048, (tokens,), generator=g).tolist(), [tokens - 1])])
        eng.finish(count[0])

    _timeline(step, 3, f"prefill step, one prompt of {tokens} tokens, {layers} Scout-sized layers")


CASES = {"sweep": case_sweep, "decode_timeline": case_decode_timeline, "prefill_timeline": case_prefill_timeline, "decode_attention": case_decode_attention, "decode_attention_fused": case_decode_attention_fused, "expert_gemv": case_expert_gemv, "expert_tc": case_expert_tc,
         "prefill_attention": case_prefill_attention, "decode_step": case_decode_step, "prefill_step": case_prefill_step}


if __name__ == "__main__":
    sys.exit(main())

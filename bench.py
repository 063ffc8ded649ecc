#!/usr/bin/env python3
"""Decode and prefill throughput of the Llama 4 engine on one B200, with roofline fractions.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--batch B] [--context C]

Default: the Scout-layer-sized 16-layer model with seeded random bfloat16 weights, batch 8,
8,192-token contexts. Token ids are uniform over the vocabulary; the caches of the decode
measurements are filled with seeded noise instead of being produced by a prefill (the bytes a
decode step reads are the same). One JSON line is printed:
  value            decoded tokens per second at the default batch, timed on the device
  e2e              the same through hi_b200.LLM (scheduler, sampler, host tokens in and out)
  prefill          one 2,048-token prompt in one step; frac = flops / time / bf16 peak
  roofline         bytes a decode step must read (every weight it uses once + live cache) / time
  points           decode tokens per second at batch 1 and 64
The reference (PipeNetwork/hi) runs Llama 4 only through Apple MLX/Metal, so ``--impl
reference`` reports that it is unavailable here.
"""
from __future__ import annotations

import argparse
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


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="scout", choices=sorted(MODELS))
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--points", default="1,64")
    ap.add_argument("--skip-prefill", action="store_true")
    args = ap.parse_args(argv)
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
    from hi_b200.engine.core import Engine, StepEntry
    from hi_b200.kernels import ops
    from hi_b200.sampling import SamplingParams

    pk = peaks()
    base_cfg, FULL_LAYERS = MODELS[args.model]
    if args.layers is None:
        args.layers = FULL_LAYERS
    cfg = dict(base_cfg, num_hidden_layers=args.layers)
    points = sorted({int(p) for p in args.points.split(",") if p} | {args.batch})
    max_batch = max(points)
    page = 64
    ctx_len = args.context
    cache_tokens = max_batch * (ctx_len + page) + args.prefill_tokens + 4 * page
    # rotary layers keep one attention chunk per request (plus the pages being written)
    chunk_tokens = max_batch * (min(ctx_len, cfg["attention_chunk_size"]) + 2 * page) + args.prefill_tokens + 4 * page
    t0 = time.time()
    engine = Engine.from_config(cfg, seed=0, std=0.02, dtype="bfloat16", kv_page_size=page,
                                kv_cache_tokens=cache_tokens, windowed_cache_tokens=chunk_tokens,
                                max_active_requests=max_batch + 2)
    torch.cuda.synchronize()
    load_s = time.time() - t0
    gen = torch.Generator(device="cuda").manual_seed(1)
    for view in engine.cache.views.values():            # seeded noise instead of a prefill
        if view.k_pages is not None:
            view.k_pages.normal_(0.0, 1.0, generator=gen)
            view.v_pages.normal_(0.0, 1.0, generator=gen)
    vocab = cfg["vocab_size"]
    cpu_gen = torch.Generator().manual_seed(2)
    sampler = ClockSampler()
    sampler.start()

    def timed_decode(batch):
        """W + K single-token steps of `batch` requests whose contexts end at ctx_len."""
        total = args.warmup + args.steps + 1
        ids = [f"d{batch}-{i}" for i in range(batch)]
        for rid in ids:
            engine.assume_cached(rid, ctx_len - total)
        toks = torch.randint(0, vocab, (total, batch), generator=cpu_gen).tolist()
        # one step with a tap to count the distinct experts a step touches, then the warm-up
        # steps (the first is eager, the second captures the CUDA graph of this shape)
        taps = {}
        engine.step([StepEntry(r, [toks[total - 1][i]], [0]) for i, r in enumerate(ids)],
                    tap=lambda n, t: taps.__setitem__(n, t))
        distinct = {int(n.split(".")[2]): len(set(t.flatten().tolist())) for n, t in taps.items()
                    if n.endswith("router_ids")}
        for s in range(args.warmup):
            engine.step([StepEntry(r, [toks[s][i]], [0]) for i, r in enumerate(ids)])
        torch.cuda.synchronize()
        launches0 = ops.LAUNCHES[0]
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for s in range(args.warmup, total - 1):
            logits = engine.step([StepEntry(r, [toks[s][i]], [0]) for i, r in enumerate(ids)])
        end.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(end) / args.steps
        launches = ops.LAUNCHES[0] - launches0
        for rid in ids:
            engine.finish(rid)
        return ms, launches, distinct

    def decode_bytes(batch, distinct):
        wb, kv, _ = model_bytes_and_flops(engine.model, distinct, ctx_len)
        return wb + batch * kv

    results = {}
    for b in points:
        ms, launches, distinct = timed_decode(b)
        results[b] = {"ms": ms, "tok_s": b * 1000.0 / ms, "launches": launches,
                      "distinct": (sum(distinct.values()) / len(distinct) if distinct else 0.0),
                      "bytes": decode_bytes(b, distinct)}
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
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights N(0,0.02), uniform random token ids, noise-filled KV cache",
        "config": {"model": f"llama4-{args.model}-layers", "layers": args.layers, "layers_full": FULL_LAYERS,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "experts": cfg["num_local_experts"], "top_k": cfg["num_experts_per_tok"],
                   "expert_inter": cfg["intermediate_size"], "mlp_inter": cfg["intermediate_size_mlp"],
                   "moe_every": cfg.get("interleave_moe_layer_step", 1), "vocab": vocab, "chunk": cfg["attention_chunk_size"],
                   "global_batch": args.batch, "seq_len": ctx_len, "page": page, "parallelism": "single-gpu",
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
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())

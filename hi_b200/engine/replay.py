"""Trace replay: feed given token ids through the model step by step and write logits.

It samples nothing and has no forward pass, cache or loader of its own: it builds the same
:class:`~hi_b200.engine.core.Engine` that generation uses and calls its ``step``. (The
reference's closest tools: ``hi-local qwen-cpu --tokens … --include-logits``,
crates/hi-local/src/main.rs:60-83, and the captured-batch replay of
crates/hi-mlx/src/models.rs:11709-11831.)

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N
              [--page-size P] [--num-pages-global G] [--num-pages-chunk K] [--max-live R] [--cpu]

``--max-tokens`` sizes every page pool (rounded up to whole pages); ``--num-pages-global`` and
``--num-pages-chunk`` size the pool of the layers that keep every key and the pool of the
windowed layers on their own, so a trace can be driven into the exhaustion of one of them.

``--cpu`` (with ``--dtype float32``) answers the same trace from the CPU reference execution
instead: no GPU, no cache and no step function, every request recomputed whole by the host
runtime's plain loops whenever logits of it are wanted (the reference's ``--execution
cpu-reference`` beside its GPU path, crates/hi-cuda/src/lib.rs:205-226). It is the third arm that
a trace can be held against, and it runs where there is no GPU.

Standard input: one JSON object per line,
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step that wants logits, ``OUT/<step>.f32`` holds them as little-endian float32
[wanted, vocab] in the order of the entries and of ``want``. After every step a line
``done <step>`` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

PAGE_SIZE = 64
MAX_LIVE_REQUESTS = 8
PAGE_SIZES = (8, 16, 32, 64, 128)      # the reference's page sizes and one larger (crates/hi-cuda/src/lib.rs:634-636)


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="trace_run", description="Replay a token trace and write logits.")
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    p.add_argument("--out", required=True, help="folder for <step>.f32 files")
    p.add_argument("--max-tokens", type=int, required=True,
                   help="most tokens live requests hold at any time (each rounded up to the page size)")
    p.add_argument("--device", default="cuda:0")
    p.add_argument("--page-size", type=int, default=PAGE_SIZE, choices=PAGE_SIZES, help="tokens per cache page")
    p.add_argument("--num-pages-global", type=int, default=None,
                   help="pages of the pool of layers that keep every key (default: --max-tokens in pages)")
    p.add_argument("--num-pages-chunk", type=int, default=None,
                   help="pages of the pool of windowed layers (default: --max-tokens in pages)")
    p.add_argument("--max-live", type=int, default=MAX_LIVE_REQUESTS, help="requests that may be live at a time")
    p.add_argument("--cpu", action="store_true",
                   help="the CPU reference execution (float32, whole sequences recomputed, no cache) instead of the engine")
    p.add_argument("--dump-taps", action="store_true",
                   help="debug: also write <step>.taps.json with the integer tensors parts report "
                        "(the router's expert choices, in the step's flat token order)")
    return p


def run(args, stdin=None, stdout=None) -> int:
    stdin = stdin or sys.stdin
    stdout = stdout or sys.stdout
    os.makedirs(args.out, exist_ok=True)
    if args.cpu:
        return _run_on_cpu(args, stdin, stdout)
    from .core import Engine, StepEntry

    page = args.page_size
    if args.max_tokens < 1 or args.max_live < 1 or (args.num_pages_global or 1) < 1 or (args.num_pages_chunk or 1) < 1:
        raise SystemExit("trace_run: --max-tokens, --max-live and the page counts must be positive")
    # each request's count is rounded up to 64 tokens (to the page, where that is larger)
    capacity = -(-args.max_tokens // max(page, PAGE_SIZE)) * max(page, PAGE_SIZE)
    engine = Engine.from_dir(args.model, dtype=args.dtype, device=args.device, kv_page_size=page,
                             kv_cache_tokens=args.num_pages_global * page if args.num_pages_global else capacity,
                             windowed_cache_tokens=args.num_pages_chunk * page if args.num_pages_chunk else capacity,
                             max_active_requests=args.max_live)
    for line in stdin:
        line = line.strip()
        if not line:
            continue
        obj = json.loads(line)
        step = obj["step"]
        entries = [StepEntry(e["id"], e["tokens"], e.get("want", [])) for e in obj.get("entries", [])]
        taps = {}
        tap = (lambda name, t: taps.__setitem__(name, t.detach().to("cpu").tolist())) if args.dump_taps else None
        logits = engine.step(entries, tap=tap) if entries else None
        if args.dump_taps:
            with open(os.path.join(args.out, f"{step}.taps.json"), "w") as f:
                json.dump(taps, f)
        if logits is not None:
            arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
            tmp = os.path.join(args.out, f"{step}.f32.tmp")
            arr.tofile(tmp)
            os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
        for rid in obj.get("end", []):
            engine.finish(rid)
        print(f"done {step}", file=stdout, flush=True)
    return 0


def _run_on_cpu(args, stdin, stdout) -> int:
    """The same protocol, answered by :class:`~hi_b200.engine.cpu_reference.CpuReference`: it keeps
    each live request's tokens and runs them whole for every step that wants logits of it."""
    import numpy as np

    from .cpu_reference import CpuReference

    if args.dtype != "float32":
        raise SystemExit("trace_run: --cpu is the float32 reference execution; give --dtype float32")
    if args.dump_taps:
        raise SystemExit("trace_run: --dump-taps reports what the engine's parts see; it has no meaning with --cpu")
    ref = CpuReference.from_dir(args.model)
    held = {}
    for line in stdin:
        line = line.strip()
        if not line:
            continue
        obj = json.loads(line)
        step, rows = obj["step"], []
        for e in obj.get("entries", []):
            if len(held) >= args.max_live and e["id"] not in held:
                raise SystemExit(f"trace_run: more than --max-live {args.max_live} requests are live")
            tokens = held.setdefault(e["id"], [])
            first = len(tokens)
            tokens.extend(int(t) for t in e["tokens"])
            want = [first + int(w) for w in e.get("want", [])]
            if any(not first <= w < len(tokens) for w in want):
                raise SystemExit(f"trace_run: step {step}, request {e['id']!r}: a wanted place is outside its tokens")
            if want:
                rows.append(ref.forward(tokens, want=want).numpy())
        if rows:
            arr = np.concatenate(rows, axis=0).astype("<f4", copy=False)
            tmp = os.path.join(args.out, f"{step}.f32.tmp")
            arr.tofile(tmp)
            os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
        for rid in obj.get("end", []):
            held.pop(rid, None)
        print(f"done {step}", file=stdout, flush=True)
    return 0


def main(argv=None) -> int:
    return run(build_parser().parse_args(argv))


if __name__ == "__main__":
    sys.exit(main())

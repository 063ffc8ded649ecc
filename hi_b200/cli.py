"""Command line, in the manner of the reference's ``hi-local`` (crates/hi-local/src/main.rs:20-84):

    python -m hi_b200 inspect MODEL_PATH
    python -m hi_b200 run MODEL_PATH (--tokens "1,2,3" | --tokens-file F | --prompt TEXT) [--max-tokens N] [--top-k 5] [--temperature T]
                          [--top-p P] [--seed S] [--include-logits] [--dtype bfloat16|float32]
                          [--max-batch-size 8] [--max-batched-tokens 8192] [--kv-page-size 64]
                          [--random-weights [--weights-seed S] [--weights-std 0.02]] [--cpu]
    python -m hi_b200 random-weights CONFIG_JSON OUT_DIR [--seed S] [--std 0.02]

``run --cpu`` runs the float32 CPU reference (``hi_b200/engine/cpu_reference.py``), as the
reference's ``--execution cpu-reference`` does (crates/hi-cuda/src/lib.rs:205-226).
``run`` is the counterpart of ``hi-local qwen-cpu``: token ids in, pretty JSON out with the same
fields (crates/hi-cuda/src/qwen_cpu.rs:62-81); ``--top-k`` is the number of top logits shown,
as there. There is no ``serve``: servers are outside this engine.
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import List


def parse_token_ids(value: str) -> List[int]:
    """Comma- or whitespace-separated ids (crates/hi-local/src/main.rs:466-475)."""
    out = []
    for part in value.replace(",", " ").split():
        if not part.isdigit():
            raise ValueError(f"invalid token id {part!r}")
        out.append(int(part))
    return out


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="hi_b200", description="decoder inference on one B200; the model class is chosen by config.json")
    sub = p.add_subparsers(dest="command", required=True)
    i = sub.add_parser("inspect", help="inspect a model folder")
    i.add_argument("model_path")
    r = sub.add_parser("run", help="run token ids through the model and generate")
    r.add_argument("model_path")
    r.add_argument("--tokens")
    r.add_argument("--tokens-file")
    r.add_argument("--prompt", help="text instead of token ids; needs tokenizer.json in the model folder")
    r.add_argument("--max-tokens", type=int, default=0)
    r.add_argument("--top-k", type=int, default=5)
    r.add_argument("--temperature", type=float, default=0.0)
    r.add_argument("--top-p", type=float, default=1.0)
    r.add_argument("--seed", type=int, default=None)
    r.add_argument("--include-logits", action="store_true")
    r.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    r.add_argument("--max-batch-size", type=int, default=8)
    r.add_argument("--max-active-requests", type=int, default=None)
    r.add_argument("--max-batched-tokens", type=int, default=8192)
    r.add_argument("--kv-page-size", type=int, default=64)
    r.add_argument("--cpu", action="store_true",
                   help="run the float32 CPU reference (plain C++ loops, whole sequences, no GPU) instead of the engine")
    r.add_argument("--random-weights", action="store_true",
                   help="MODEL_PATH is a config.json (or a folder with one); weights are seeded random numbers")
    r.add_argument("--weights-seed", type=int, default=0)
    r.add_argument("--weights-std", type=float, default=0.02)
    w = sub.add_parser("random-weights", help="write a model folder with seeded random weights")
    w.add_argument("config_json")
    w.add_argument("out_dir")
    w.add_argument("--seed", type=int, default=0)
    w.add_argument("--std", type=float, default=0.02)
    return p


def cmd_inspect(args) -> int:
    import torch

    from .config.registry import load_architecture
    from .parts.model import Model
    from .weights.loader import WeightError, check_names
    from .weights.safetensors_io import Checkpoint

    arch, cfg, raw = load_architecture(args.model_path)
    spec = arch.build_spec(cfg)
    model = Model(spec, torch.bfloat16, "cpu")
    specs = model.tensor_specs()
    params = sum(int(torch.Size(s.shape).numel()) for s in specs if s.init != "absent")
    report = {
        "architecture": arch.name, "architectures": list(getattr(cfg, "architectures", ())),
        "layers": [{"layer": i, "mixer": l.mixer.kind, "window": l.mixer.params.get("window"),
                    "position": (l.mixer.params.get("position") or {}).kind if l.mixer.params.get("position") else None,
                    "feed_forward": l.feed_forward.kind} for i, l in enumerate(spec.layers)],
        "schedule": [e.layer for e in spec.schedule],
        "parameters": params, "weight_bytes_bf16": 2 * params,
        "kv_bytes_per_token_bf16": sum(2 * 2 * cs.kv_heads * cs.head_dim for cs in model.cache_specs.values() if cs),
        "config": {k: v for k, v in vars(cfg).items() if k != "raw"},
    }
    try:
        ckpt = Checkpoint(args.model_path)
        names = {}
        for n in ckpt.names():
            m = arch.normalize_tensor_name(n)
            if m is not None:
                names[m] = ckpt.describe(n)[1]
        if arch.derive_tensors is not None:          # tensors stored in another layout of the same weights
            for name, d in arch.derive_tensors(dict(names)).items():
                names[name] = d.shape
                for src in d.sources:
                    names.pop(src, None)
        check_names(specs, names, args.model_path)
        report["tensors"] = {"count": len(names), "status": "ok"}
    except (WeightError, ValueError) as e:
        report["tensors"] = {"status": "error", "message": str(e)}
    print(json.dumps(report, indent=2, default=str))
    return 0 if report["tensors"]["status"] == "ok" else 1


def cmd_run(args) -> int:
    import os

    from .tokenizer import TokenizerRuntime

    if sum(bool(v) for v in (args.tokens, args.tokens_file, args.prompt)) != 1:
        raise SystemExit("provide exactly one of --tokens, --tokens-file and --prompt")
    tokenizer = TokenizerRuntime.load(args.model_path) if os.path.isdir(args.model_path) else None
    if args.prompt:
        if tokenizer is None:
            raise SystemExit("--prompt needs tokenizer.json in the model folder and the `tokenizers` package")
        tokens = tokenizer.encode(args.prompt)
    else:
        tokens = parse_token_ids(args.tokens if args.tokens else open(args.tokens_file).read())
    if not tokens:
        raise SystemExit("the prompt must include at least one token")
    args.tokenizer = tokenizer
    if args.cpu:
        return _run_on_cpu(args, tokens)
    import torch

    from .engine.core import StepEntry
    from .engine.generate import LLM
    from .kernels import ops
    from .sampling.sampler import SamplingParams

    model = args.model_path
    if args.random_weights:
        # MODEL_PATH names a config.json (or a folder with one): weights are generated on the device
        import os

        path = os.path.join(model, "config.json") if os.path.isdir(model) else model
        with open(path) as f:
            model = json.load(f)
    llm = LLM(model, random_seed=args.weights_seed, random_std=args.weights_std, dtype=args.dtype, max_batch_size=args.max_batch_size,
              max_active_requests=args.max_active_requests, max_batched_tokens=args.max_batched_tokens,
              kv_page_size=args.kv_page_size,
              kv_cache_tokens=max(args.max_batched_tokens, len(tokens) + args.max_tokens + args.kv_page_size))
    logits = llm.engine.step([StepEntry("inspect", tokens, [len(tokens) - 1])])[0]
    llm.engine.finish("inspect")
    next_token = int(ops.sample_rows(logits[None].contiguous(), None, None)[0])     # the lowest id on ties
    # the largest logits, ties by id: everything not below the k-th value is ranked on the host
    k = min(max(args.top_k, 0), logits.numel())
    top = []
    if k > 0:
        kth = torch.topk(logits, k).values[-1]
        ids = (logits >= kth).nonzero().flatten()
        top = sorted(zip(ids.tolist(), logits[ids].tolist()), key=lambda p: (-p[1], p[0]))[:k]
    generated: List[int] = []
    if args.max_tokens > 0:
        out = llm.generate([tokens], SamplingParams(max_tokens=args.max_tokens, temperature=args.temperature,
                                                    top_p=args.top_p, seed=args.seed))[0]
        generated = out.token_ids
    result = {
        "backend": f"hi_b200-cuda-{args.dtype}", "input_tokens": tokens, "next_token": next_token,
        "next_text": _text(args, [next_token]), "generated_tokens": generated, "generated_text": _text(args, generated),
        "top_logits": [{"token_id": i, "token": _token(args, i), "logit": v} for i, v in top],
        "logit_count": logits.numel(),
    }
    if args.include_logits:
        result["logits"] = logits.cpu().tolist()
    print(json.dumps(result, indent=2))
    return 0


def _text(args, tokens) -> str:
    """Text of token ids where the model folder has a tokenizer, else the empty string."""
    tok = getattr(args, "tokenizer", None)
    return tok.decode(tokens) if tok is not None and tokens else ""


def _token(args, token_id: int):
    tok = getattr(args, "tokenizer", None)
    return tok.token(token_id) if tok is not None else None


def _run_on_cpu(args, tokens: List[int]) -> int:
    """``run --cpu``: the same JSON from the float32 CPU reference."""
    import numpy as np

    from .engine.cpu_reference import CpuReference
    from .sampling.sampler import SamplingParams

    if args.random_weights:
        raise SystemExit("--cpu reads a model folder; write one with `random-weights` first")
    if args.dtype != "float32":
        print("note: the CPU reference computes in float32 whatever --dtype says", file=sys.stderr)
    ref = CpuReference.from_dir(args.model_path)
    row = ref.forward(tokens, want=[len(tokens) - 1])[0].numpy()
    k = min(max(args.top_k, 0), row.size)
    order = np.lexsort((np.arange(row.size), -row))[:k]
    generated: List[int] = []
    if args.max_tokens > 0:
        generated = ref.generate(tokens, args.max_tokens, SamplingParams(
            max_tokens=args.max_tokens, temperature=args.temperature, top_p=args.top_p, seed=args.seed),
            eos_token_ids=ref.model.spec.eos_token_ids)
    result = {
        "backend": "hi_b200-cpu-reference-float32", "input_tokens": tokens, "next_token": int(np.argmax(row)),
        "next_text": _text(args, [int(np.argmax(row))]), "generated_tokens": generated, "generated_text": _text(args, generated),
        "top_logits": [{"token_id": int(i), "token": _token(args, int(i)), "logit": float(row[i])} for i in order],
        "logit_count": int(row.size),
    }
    if args.include_logits:
        result["logits"] = row.tolist()
    print(json.dumps(result, indent=2))
    return 0


def cmd_random_weights(args) -> int:
    from .weights.loader import write_random_model

    with open(args.config_json) as f:
        config = json.load(f)
    write_random_model(config, args.out_dir, args.seed, args.std)
    print(json.dumps({"model_path": args.out_dir, "seed": args.seed, "std": args.std}))
    return 0


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    return {"inspect": cmd_inspect, "run": cmd_run, "random-weights": cmd_random_weights}[args.command](args)


if __name__ == "__main__":
    sys.exit(main())

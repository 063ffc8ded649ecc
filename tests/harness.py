"""Helpers of the tests: model folders, the plain model as oracle, traces and their replay."""
from __future__ import annotations

import json
import os
import random
import subprocess
import sys
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

import plain_llama4 as plain

ROOT = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

# tolerances: max |engine - plain| / max |plain| over the compared logits
TOL_F32 = 2e-5
TOL_BF16 = 2.5e-2
# a bfloat16 engine may pick another expert than the plain model only where the plain model's k-th and
# (k+1)-th router logits are closer than this fraction of the root mean square of the layer's router
# logits over the sequence (the router reads the norm's float32 output; what reaches it in reduced
# precision is the sub-layers' bfloat16 outputs summed in the residual stream, an error proportional
# to the size of the logits, not to one token's). Measured over 83,000 decisions of the four tiny
# models at two weight scales and up to 1,040 tokens: the largest such fraction among differing
# choices was 0.040 (0.011 to 0.020 for seven of the eight models).
ROUTING_MARGIN = 0.06


def make_model(path: str, cfg: dict, seed: int, std: float = 0.08, overrides=None) -> str:
    from hi_b200.weights import write_random_model

    return write_random_model(cfg, path, seed=seed, std=std, overrides=overrides)


def read_weights(model_dir: str) -> Dict[str, torch.Tensor]:
    """Independent of hi_b200's reader: the safetensors package."""
    from safetensors import safe_open

    out = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            out[k] = f.get_tensor(k)
    return out


def vocab_of(cfg: dict) -> int:
    return plain.text_config(cfg)["vocab_size"]


def random_tokens(cfg: dict, n: int, seed: int) -> List[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab_of(cfg)) for _ in range(n)]


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    return float((got.float().cpu() - want.float()).abs().max() / (want.float().abs().max() + 1e-12))


# --------------------------------------------------------------------------- traces
# A trace is a list of steps; a step is (entries, end) with entries = [(request id, tokens, want)].
Step = Tuple[List[Tuple[Hashable, List[int], List[int]]], List[Hashable]]


def trace_whole(requests: Dict[Hashable, List[int]]) -> List[Step]:
    """Each request alone and whole: one step, logits at every position."""
    return [([(rid, toks, list(range(len(toks))))], [rid]) for rid, toks in requests.items()]


def trace_tail_decode(requests: Dict[Hashable, List[int]], tail: int = 32) -> List[Step]:
    """Most of each request in one step, the last ``tail`` tokens one by one."""
    steps: List[Step] = []
    for rid, toks in requests.items():
        head = max(len(toks) - tail, min(2, len(toks)))
        steps.append(([(rid, toks[:head], list(range(head)))], []))
        for i in range(head, len(toks)):
            steps.append(([(rid, [toks[i]], [0])], []))
        steps[-1] = (steps[-1][0], [rid])
    return steps


def trace_portions(requests: Dict[Hashable, List[int]], sizes: Sequence[int] = (13, 7, 2, 5, 3, 2, 31, 2, 17, 1, 9, 64, 2)) -> List[Step]:
    """Each request alone, in portions of changing size, down to two tokens (and one)."""
    steps: List[Step] = []
    for k, (rid, toks) in enumerate(requests.items()):
        pos, i = 0, k
        while pos < len(toks):
            n = min(sizes[i % len(sizes)], len(toks) - pos)
            i += 1
            steps.append(([(rid, toks[pos:pos + n], list(range(n)))], []))
            pos += n
        steps[-1] = (steps[-1][0], [rid])
    return steps


def trace_mixed(requests: Dict[Hashable, List[int]], max_tokens: int, page: int, seed: int = 0, max_live: int = 4,
                prefill_len: Optional[Dict[Hashable, int]] = None) -> List[Step]:
    """Up to ``max_live`` requests at a time; portions of some beside single decoded tokens of
    others; a request starts as soon as the tokens held by live requests (each rounded up to
    ``page``) leave room for all of it, so pages of finished requests are used again."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live: Dict[Hashable, Tuple[List[int], int]] = {}      # rid -> (tokens, done)
    steps: List[Step] = []
    rounded = lambda n: -(-n // page) * page
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting[0]
            held = sum(rounded(len(t)) for t, _ in live.values())
            if held + rounded(len(toks)) > max_tokens:
                break
            live[rid] = (toks, 0)
            waiting.pop(0)
        if not live:
            raise ValueError("max_tokens is too small for the next request")
        entries, end = [], []
        for rid in list(live):
            toks, done = live[rid]
            pl = (prefill_len or {}).get(rid, max(2, len(toks) - 24))
            if rng.random() < 0.2 and len(live) > 1:
                continue                                    # left out of this step, goes on later
            if done < pl:
                n = min(rng.choice([2, 3, 5, 8, 13, 21, 40]), pl - done)
            else:
                n = 1
            entries.append((rid, toks[done:done + n], list(range(n))))
            done += n
            live[rid] = (toks, done)
            if done == len(toks):
                end.append(rid)
                del live[rid]
        if entries:
            steps.append((entries, end))
    return steps


def trace_json(steps: List[Step]) -> str:
    lines = []
    for i, (entries, end) in enumerate(steps):
        lines.append(json.dumps({"step": i, "entries": [{"id": str(r), "tokens": t, "want": w} for r, t, w in entries],
                                 "end": [str(r) for r in end]}))
    return "\n".join(lines) + "\n"


def collect(steps: List[Step], per_step_logits: Dict[int, np.ndarray]) -> Dict[Hashable, Dict[int, np.ndarray]]:
    """{request: {position: logits row}} from the per-step outputs."""
    pos: Dict[Hashable, int] = {}
    out: Dict[Hashable, Dict[int, np.ndarray]] = {}
    for i, (entries, _end) in enumerate(steps):
        row = 0
        for rid, toks, want in entries:
            start = pos.get(rid, 0)
            for w in want:
                out.setdefault(rid, {})[start + w] = per_step_logits[i][row]
                row += 1
            pos[rid] = start + len(toks)
    return out


def replay_subprocess(model_dir: str, dtype: str, steps: List[Step], max_tokens: int, out_dir: str,
                      vocab: int, timeout: int = 600, dump_taps: bool = False, extra: Sequence[str] = ()):
    """Run bin/trace_run as a user would and read back its files. With ``dump_taps`` also
    returns the router's choices per request ({request: {layer prefix: ids [T, k]}})."""
    os.makedirs(out_dir, exist_ok=True)
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens)] + (["--dump-taps"] if dump_taps else []) + list(extra)
    proc = subprocess.run(cmd, input=trace_json(steps), capture_output=True, text=True, timeout=timeout)
    assert proc.returncode == 0, f"trace_run failed ({proc.returncode}):\n{proc.stdout[-2000:]}\n{proc.stderr[-4000:]}"
    done = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
    assert [int(l.split()[1]) for l in done] == list(range(len(steps))), "trace_run did not report every step in order"
    per_step = {}
    for i, (entries, _e) in enumerate(steps):
        n = sum(len(w) for _r, _t, w in entries)
        path = os.path.join(out_dir, f"{i}.f32")
        if n:
            data = np.fromfile(path, dtype="<f4")
            assert data.size == n * vocab, f"step {i}: {data.size} floats for {n} wanted rows of {vocab}"
            per_step[i] = data.reshape(n, vocab)
        else:
            assert not os.path.exists(path), f"step {i} wanted nothing but wrote a file"
    got = collect(steps, per_step)
    if not dump_taps:
        return got
    routing: Dict[Hashable, Dict[str, List[torch.Tensor]]] = {}
    for i, (entries, _e) in enumerate(steps):
        with open(os.path.join(out_dir, f"{i}.taps.json")) as f:
            taps = json.load(f)
        for name, ids in taps.items():
            if not name.endswith(".router_ids"):
                continue
            ids = torch.tensor(ids)
            cursor = 0
            for rid, toks, _w in entries:
                routing.setdefault(rid, {}).setdefault(name[: -len(".router_ids")], []).append(
                    ids[cursor: cursor + len(toks)])
                cursor += len(toks)
    forced = {rid: {n: torch.cat(parts) for n, parts in layers.items()} for rid, layers in routing.items()}
    return got, forced


def replay_in_process(engine, steps: List[Step], record_routing: bool = False, forced_routing=None):
    """Drive Engine.step directly; optionally gather the router's choices per request, or hand
    choices back (``forced_routing`` {request: {layer prefix: ids [T, k]}} by position)."""
    from hi_b200.engine.core import StepEntry

    per_step = {}
    routing: Dict[Hashable, Dict[str, List[torch.Tensor]]] = {}
    fed: Dict[Hashable, int] = {}
    for i, (entries, end) in enumerate(steps):
        taps: Dict[str, torch.Tensor] = {}
        tap = (lambda name, t: taps.__setitem__(name, t.clone())) if record_routing else None
        forced = None
        if forced_routing is not None:
            names = sorted({n for r, _t, _w in entries for n in forced_routing.get(r, {})})
            forced = {f"{n}.router_ids": torch.cat([forced_routing[r][n][fed.get(r, 0): fed.get(r, 0) + len(t)]
                                                    for r, t, _w in entries]).to(torch.int32) for n in names}
        for r, t, _w in entries:
            fed[r] = fed.get(r, 0) + len(t)
        logits = engine.step([StepEntry(r, t, w) for r, t, w in entries], tap=tap, forced=forced)
        if logits is not None:
            per_step[i] = logits.float().cpu().numpy()
        if record_routing:
            for name, ids in taps.items():
                if not name.endswith(".router_ids"):
                    continue
                ids = ids.cpu()
                cursor = 0
                for rid, toks, _w in entries:
                    routing.setdefault(rid, {}).setdefault(name[: -len(".router_ids")], []).append(
                        ids[cursor: cursor + len(toks)])
                    cursor += len(toks)
        for rid in end:
            engine.finish(rid)
        engine.manager.check_invariants()
    got = collect(steps, per_step)
    forced = {rid: {name: torch.cat(parts) for name, parts in layers.items()} for rid, layers in routing.items()}
    return got, forced


def compare_with_plain(cfg: dict, weights, requests: Dict[Hashable, List[int]], got, tol: float,
                       forced=None, what: str = "", margin: float = 0.0) -> None:
    """Every wanted row of every request against the plain model; names the first wrong token.

    ``forced``: the engine's own expert choices (reduced precision may pick the other of two
    nearly equal router logits; the logits are then compared given that choice). The choices
    themselves must equal the plain model's wherever its k-th and (k+1)-th logits are more
    than ``margin`` (a fraction of the root mean square of the layer's router logits) apart."""
    for rid, toks in requests.items():
        records = {}
        ref = plain.forward(cfg, weights, toks, forced_routing=(forced or {}).get(rid),
                            record=lambda name, ids, gap: records.__setitem__(name, (ids, gap)))
        for name, ids in ((forced or {}).get(rid) or {}).items():
            own, gap = records[name]
            differs = (own.sort(-1).values != ids.long().sort(-1).values).any(-1)
            clear = differs & (gap > margin)
            assert not bool(clear.any()), (
                f"{what}: request {rid!r}, {name}: expert choice differs at positions "
                f"{clear.nonzero().flatten().tolist()[:8]} where the plain model's margin is clear")
        scale = float(ref.abs().max())
        rows = got.get(rid, {})
        assert rows, f"{what}: no logits came back for request {rid!r}"
        for p in sorted(rows):
            err = float(np.abs(rows[p] - ref[p].numpy()).max()) / scale
            assert np.isfinite(err) and err <= tol, (
                f"{what}: request {rid!r} first differs at position {p} of {len(toks)}: rel err {err:.3e} > {tol:.1e}")

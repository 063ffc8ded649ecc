"""Writes tests/golden/plain_tiny.json: outputs of the plain implementation (tests/plain_llama4.py)
on the tiny random models, to pin it against later edits.

The reference's own Llama 4 code cannot run here (Apple MLX/Metal only, no Rust toolchain), so
these numbers rest on the plain implementation's formulas, not on the reference's outputs.

    python tests/golden/make_golden.py
"""
import json
import os
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, ".."))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

import harness as h  # noqa: E402
import plain_llama4 as plain  # noqa: E402
from tiny_configs import TINY_A, TINY_B, TINY_C  # noqa: E402


def main():
    out = {}
    for name, cfg in (("A", TINY_A), ("B", TINY_B), ("C", TINY_C)):
        with tempfile.TemporaryDirectory() as d:
            h.make_model(d, cfg, seed=11, std=0.08)
            w = h.read_weights(d)
        toks = h.random_tokens(cfg, 60, seed=1)
        logits = plain.forward(cfg, w, toks)
        out[name] = {
            "tokens": toks,
            "argmax": [int(r.argmax()) for r in logits],
            "rows": {str(p): [round(float(v), 6) for v in logits[p][:12]] for p in (0, 1, 15, 16, 31, 32, 33, 59)},
            "checksum": round(float(logits.double().abs().sum()), 4),
        }
    with open(os.path.join(HERE, "plain_tiny.json"), "w") as f:
        json.dump(out, f, indent=1)


if __name__ == "__main__":
    main()

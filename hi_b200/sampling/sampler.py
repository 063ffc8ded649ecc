"""Sampling: greedy, temperature, and ranked (top-k / top-p), per request.

Greedy and temperature-only rows are sampled on the GPU in one launch
(``hi_b200/csrc/sampling.cu``); ranked rows by a second kernel that follows the host sampler's rule
(the reference ranks on the host by default: crates/hi-cuda/src/kernels.cu:8041-8072 and the
comment above it; host sampler crates/hi-cuda/src/qwen_cpu.rs:3657-3732,
crates/hi-mlx/src/generate.rs:50-110). :func:`ranked_sample` is that rule on the host; it takes the
rows the kernel hands back (more than 4,096 candidates).
Each request owns its generator and draws exactly one uniform per sampled token, so its
stream does not depend on what else is in the batch (crates/hi-cuda/src/lib.rs:5658-5662).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..kernels import ops

DEFAULT_SEED = 0x4849          # crates/hi-mlx/src/models.rs:576-581
_MASK = 0xFFFFFFFFFFFFFFFF


class Lcg:
    """The reference's generator (crates/hi-mlx/src/generate.rs:123-146)."""

    def __init__(self, seed: int):
        self.state = (int(seed) ^ 0x9E3779B97F4A7C15) & _MASK

    def next_f32(self) -> float:
        self.state = (self.state * 6364136223846793005 + 1442695040888963407) & _MASK
        return float(self.state >> 40) / float(1 << 24)


@dataclass
class SamplingParams:
    """Names and meanings as the reference's request (crates/hi-local-core/src/backend.rs:12-24)."""

    max_tokens: int = 16
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: Optional[int] = None
    seed: Optional[int] = None
    ignore_eos: bool = False
    stop_token_ids: Tuple[int, ...] = ()

    def validate(self) -> None:
        """crates/hi-cuda/src/lib.rs:3023-3036, 6869-6919."""
        if self.max_tokens < 1:
            raise ValueError("invalid_request_parameter: max_tokens must be at least 1")
        if not (self.temperature >= 0.0) or not np.isfinite(self.temperature):
            raise ValueError("invalid_request_parameter: temperature must be finite and >= 0")
        if not (0.0 <= self.top_p <= 1.0):
            raise ValueError("invalid_request_parameter: top_p must lie in [0, 1]")
        if self.top_k is not None and self.top_k <= 0:
            raise ValueError("invalid_request_parameter: top_k must be positive when given")

    @property
    def greedy(self) -> bool:
        return not (self.temperature > 0.0)

    def ranked(self, vocab: int) -> bool:
        k = self.top_k if (self.top_k and 0 < self.top_k < vocab) else vocab
        return (not self.greedy) and not (k == vocab and self.top_p >= 1.0)


def ranked_sample(row: np.ndarray, temperature: float, top_p: float, top_k: Optional[int], u: float) -> int:
    """Host sampler for top-k / top-p: softmax(l/T), sort descending with ties by id, cut to
    top-k, keep the shortest prefix whose mass reaches top_p, walk it with draw = u * kept mass."""
    z = row.astype(np.float32) / np.float32(temperature)
    w = np.exp(z - z.max(), dtype=np.float32)
    p = w / w.sum(dtype=np.float32)
    order = np.lexsort((np.arange(p.size), -p))
    if top_k and 0 < top_k < p.size:
        order = order[:top_k]
    cutoff = min(max(top_p, 0.0), 1.0)
    if 0.0 < cutoff < 1.0:
        cum = np.cumsum(p[order], dtype=np.float32)
        keep = int(np.searchsorted(cum, np.float32(cutoff), side="left")) + 1
        order = order[:max(min(keep, order.size), 1)]
    draw = np.float32(u) * p[order].sum(dtype=np.float32)
    for i in order:
        if draw <= p[i]:
            return int(i)
        draw -= p[i]
    return int(np.argmax(row))


def sample_on_host(row: np.ndarray, params: SamplingParams, rng: Lcg) -> int:
    """One token from one row of float32 logits on the host, by the rules of the kernels: the
    largest logit (the lowest id on ties) when greedy; temperature alone: weights exp(l/T - max)
    walked in vocabulary order, the first id whose running sum exceeds u * total
    (crates/hi-cuda/src/kernels.cu:7327-7352); top-k / top-p: :func:`ranked_sample`. Draws one
    uniform from ``rng`` unless greedy."""
    row = np.asarray(row, dtype=np.float32)
    if params.greedy:
        return int(np.argmax(row))                    # numpy returns the first of equal maxima
    u = rng.next_f32()
    if params.ranked(row.size):
        return ranked_sample(row, params.temperature, params.top_p, params.top_k, u)
    z = row / np.float32(params.temperature)
    w = np.exp(z - z.max(), dtype=np.float32)
    cum = np.cumsum(w, dtype=np.float32)
    i = int(np.searchsorted(cum, np.float32(u) * cum[-1], side="right"))
    return min(i, int(np.nonzero(w > 0)[0][-1]))


def sample_on_device(logits: torch.Tensor, params: Sequence[SamplingParams], rngs: Sequence[Lcg]
                     ) -> Optional[torch.Tensor]:
    """One token for each row of float32 ``logits`` [R, V], left on the device as int32 [R] (no
    wait for the GPU), or None if a row samples with top-k / top-p: the kernel that ranks them may
    hand a row back to the host, so its result has to be read at once (use :func:`sample`; no
    generator has been advanced then)."""
    rows, vocab = logits.shape
    if rows != len(params) or rows != len(rngs):
        raise ValueError("one SamplingParams and one generator per row are needed")
    if any(p.ranked(vocab) for p in params):
        return None
    if all(p.greedy for p in params):
        return ops.sample_rows(logits, None, None)
    uniforms = [0.0 if p.greedy else rng.next_f32() for p, rng in zip(params, rngs)]
    temps = [0.0 if p.greedy else float(p.temperature) for p in params]
    host = torch.tensor([temps, uniforms], dtype=torch.float32).to(logits.device, non_blocking=True)
    return ops.sample_rows(logits, host[0].contiguous(), host[1].contiguous())


def sample(logits: torch.Tensor, params: Sequence[SamplingParams], rngs: Sequence[Lcg]) -> List[int]:
    """One token for each row of float32 ``logits`` [R, V] on the device."""
    rows, vocab = logits.shape
    if rows != len(params) or rows != len(rngs):
        raise ValueError("one SamplingParams and one generator per row are needed")
    if all(p.greedy for p in params):
        return ops.sample_rows(logits, None, None).tolist()
    uniforms = [0.0 if p.greedy else rng.next_f32() for p, rng in zip(params, rngs)]
    ranked = [p.ranked(vocab) for p in params]
    # the one-launch sampler takes the greedy and the temperature-only rows (ranked rows: a
    # placeholder argmax); the ranked kernel then takes the rows with top-k / top-p
    temps = [0.0 if (p.greedy or rk) else float(p.temperature) for p, rk in zip(params, ranked)]
    rank_temps = [float(p.temperature) if rk else 0.0 for p, rk in zip(params, ranked)]
    top_ps = [float(p.top_p) for p in params]
    host = torch.tensor([temps, uniforms, rank_temps, top_ps], dtype=torch.float32).to(logits.device, non_blocking=True)
    out_dev = ops.sample_rows(logits, host[0].contiguous(), host[1].contiguous())
    if any(ranked):
        top_ks = torch.tensor([int(p.top_k or 0) for p in params], dtype=torch.int32).to(logits.device, non_blocking=True)
        ops.ranked_rows(logits, host[2].contiguous(), host[3].contiguous(), top_ks, host[1].contiguous(), out_dev)
    out = out_dev.tolist()
    for r, p in enumerate(params):
        if ranked[r] and out[r] < 0:
            # more candidates than the kernel sorts (a nearly flat distribution with a wide top-p): the host ranks
            out[r] = ranked_sample(logits[r].cpu().numpy(), p.temperature, p.top_p, p.top_k, uniforms[r])
    return out

"""The Python entry point: token ids in, generated token ids out.

The reference's request and result types (crates/hi-local-core/src/backend.rs:12-24,
161-172) carry text; this engine is token-level, so prompts and results are token ids and
the same names are kept for the rest (``max_tokens``, ``temperature``, ``top_p``, ``top_k``,
``seed``; ``prompt_tokens``, ``completion_tokens``).
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from typing import Callable, Dict, Hashable, List, Optional, Sequence, Union

import torch

from ..sampling.sampler import SamplingParams, sample
from .core import Engine, StepEntry
from .scheduler import Request, Scheduler, SchedulerConfig


@dataclass
class GenerationOutput:
    request_id: Hashable
    prompt_token_ids: List[int]
    token_ids: List[int]
    finish_reason: str
    prompt_tokens: int
    completion_tokens: int
    preemptions: int = 0


class LLM:
    """A model ready to generate: engine + scheduler + sampler.

    ``model`` is a model folder, or a config dict together with ``random_seed`` (weights are
    then generated on the device). Options are the reference's serve flags
    (crates/hi-local/src/main.rs:28-59): ``max_batch_size``, ``max_active_requests``,
    ``max_batched_tokens``, ``kv_page_size``; plus ``kv_cache_tokens`` (pool capacity) and
    ``max_prefill_portion``.
    """

    def __init__(self, model: Union[str, dict, Engine], *, dtype="bfloat16", device="cuda:0",
                 random_seed: Optional[int] = None, random_std: float = 0.02, kv_page_size: int = 64,
                 kv_cache_tokens: Optional[int] = None, windowed_cache_tokens: Optional[int] = None,
                 max_batch_size: int = 8, max_active_requests: Optional[int] = None,
                 max_batched_tokens: int = 8192, max_prefill_portion: Optional[int] = None):
        self.config = SchedulerConfig(max_batch_size=max_batch_size, max_active_requests=max_active_requests,
                                      max_batched_tokens=max_batched_tokens, max_prefill_portion=max_prefill_portion)
        self.config.validate()
        slots = max_active_requests or max_batch_size
        if isinstance(model, Engine):
            self.engine = model
        else:
            opts = dict(kv_page_size=kv_page_size, max_active_requests=slots,
                        kv_cache_tokens=kv_cache_tokens or max(max_batched_tokens, 8192),
                        windowed_cache_tokens=windowed_cache_tokens)
            if isinstance(model, dict):
                self.engine = Engine.from_config(model, seed=random_seed or 0, std=random_std, dtype=dtype,
                                                 device=device, **opts)
            else:
                self.engine = Engine.from_dir(model, dtype=dtype, device=device, **opts)
        spec = self.engine.model.spec
        self.scheduler = Scheduler(self.engine.manager, self.config, eos_token_ids=spec.eos_token_ids,
                                   max_model_len=spec.max_position_embeddings, release=self.engine.finish)
        self._ids = itertools.count()

    # ------------------------------------------------------------------ low level
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None,
                    request_id: Optional[Hashable] = None) -> Request:
        vocab = self.engine.vocab_size
        bad = [t for t in prompt if not 0 <= int(t) < vocab]
        if bad:
            raise ValueError(f"invalid_request_parameter: token ids {bad[:4]} outside 0..{vocab - 1}")
        rid = request_id if request_id is not None else f"req-{next(self._ids)}"
        req = Request(rid, [int(t) for t in prompt], params or SamplingParams())
        self.scheduler.add(req)
        return req

    def abort(self, request_id: Hashable) -> None:
        self.scheduler.abort(request_id)

    def step(self, on_token: Optional[Callable[[Hashable, int], None]] = None) -> List[Request]:
        """One scheduler iteration: plan, run the batch, sample, finish. Returns finished requests."""
        plan = self.scheduler.plan()
        if not plan.entries:
            if plan.preempted or not self.scheduler.has_work():
                return []
            raise RuntimeError("scheduler stalled: no request can take a step with the pages that are free")
        entries = [StepEntry(e.request.request_id, e.tokens, [len(e.tokens) - 1] if e.samples else [])
                   for e in plan.entries]
        logits = self.engine.step(entries)
        sampling = [e.request for e in plan.entries if e.samples]
        sampled: Dict[Hashable, int] = {}
        if sampling:
            toks = sample(logits, [r.params for r in sampling], [r.rng for r in sampling])
            sampled = {r.request_id: t for r, t in zip(sampling, toks)}
        before = {r.request_id: len(r.output) for r in sampling}
        done = self.scheduler.commit(plan, sampled)
        if on_token is not None:
            for r in sampling:
                if len(r.output) > before[r.request_id]:
                    on_token(r.request_id, r.output[-1])
        return done

    # ------------------------------------------------------------------ the call a user makes
    def generate(self, prompts: Sequence[Sequence[int]],
                 params: Union[SamplingParams, Sequence[SamplingParams], None] = None,
                 on_token: Optional[Callable[[Hashable, int], None]] = None) -> List[GenerationOutput]:
        """Generate for every prompt (lists of token ids); results in the order of the prompts."""
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompts)
        if len(params) != len(prompts):
            raise ValueError("one SamplingParams per prompt is needed")
        reqs = [self.add_request(p, sp) for p, sp in zip(prompts, params)]
        while any(r.status != "finished" for r in reqs):
            self.step(on_token)
        return [GenerationOutput(r.request_id, r.prompt, list(r.output), r.finish_reason or "", len(r.prompt),
                                 len(r.output), r.preemptions) for r in reqs]

    def stats(self) -> dict:
        s = self.engine.snapshot()
        s["scheduler"] = dict(self.scheduler.counters)
        return s


def generate(model: Union[str, dict], prompts: Sequence[Sequence[int]],
             params: Union[SamplingParams, Sequence[SamplingParams], None] = None, **options) -> List[GenerationOutput]:
    """Load ``model`` and generate once; see :class:`LLM` for the options."""
    return LLM(model, **options).generate(prompts, params)

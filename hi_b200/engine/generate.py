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

from ..sampling.sampler import SamplingParams, sample, sample_on_device
from .core import Engine, StepEntry
from .scheduler import IN_FLIGHT, Request, Scheduler, SchedulerConfig, StepPlan


@dataclass
class GenerationOutput:
    request_id: Hashable
    prompt_token_ids: List[int]
    token_ids: List[int]
    finish_reason: str
    prompt_tokens: int
    completion_tokens: int
    preemptions: int = 0


class _Launched:
    """A step that runs on the GPU while the host goes on: its plan, the requests it samples
    for, and the sampled tokens on the device, on their way to pinned host memory."""

    __slots__ = ("plan", "sampling", "tokens_dev", "tokens_host", "copied", "row_of", "status")

    def __init__(self, plan, sampling, tokens_dev, host_buffer, copied, status=None):
        self.plan, self.sampling, self.tokens_dev = plan, sampling, tokens_dev
        self.status = status                 # the step's kernel-status ticket (None: checked when it ran)
        self.row_of = {r.request_id: i for i, r in enumerate(sampling)}
        self.tokens_host = host_buffer[: tokens_dev.numel()]
        self.tokens_host.copy_(tokens_dev, non_blocking=True)
        self.copied = copied
        self.copied.record()


class _Unread:
    """A step that ran but whose samples are read at once: only its plan matters to a later look."""

    __slots__ = ("plan",)

    def __init__(self, plan):
        self.plan = plan


class LLM:
    """A model ready to generate: engine + scheduler + sampler.

    With ``lookahead`` (the default) a step is planned and launched while the step before it still
    runs: its decode tokens are taken on the device from what that step sampled, and the host reads
    the sampled tokens one step late (finished requests and ``on_token`` calls come one ``step()``
    later; a request that ends leaves one unread row in the step that was already launched). Rows
    that sample with top-k / top-p make their step wait: the kernel that ranks them may hand a row
    back to the host (more candidates than it sorts), so the host reads its result at once.

    ``model`` is a model folder, or a config dict together with ``random_seed`` (weights are
    then generated on the device). Options are the reference's serve flags
    (crates/hi-local/src/main.rs:28-59): ``max_batch_size``, ``max_active_requests``,
    ``max_batched_tokens``, ``kv_page_size``; plus ``kv_cache_tokens`` (pool capacity; by default
    nine tenths of the device memory that is free after loading) and ``max_prefill_portion``.
    """

    def __init__(self, model: Union[str, dict, Engine], *, dtype="bfloat16", device="cuda:0",
                 random_seed: Optional[int] = None, random_std: float = 0.02, kv_page_size: int = 64,
                 kv_cache_tokens: Optional[int] = None, windowed_cache_tokens: Optional[int] = None,
                 max_batch_size: int = 8, max_active_requests: Optional[int] = None,
                 max_batched_tokens: int = 8192, max_prefill_portion: Optional[int] = None, lookahead: bool = True):
        self.config = SchedulerConfig(max_batch_size=max_batch_size, max_active_requests=max_active_requests,
                                      max_batched_tokens=max_batched_tokens, max_prefill_portion=max_prefill_portion)
        self.config.validate()
        slots = max_active_requests or max_batch_size
        if isinstance(model, Engine):
            self.engine = model
        else:
            opts = dict(kv_page_size=kv_page_size, max_active_requests=slots,
                        kv_cache_tokens=kv_cache_tokens,      # None: sized from the memory that is free
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
        self.lookahead = lookahead
        self._launched: Optional[_Launched] = None       # the step whose samples the host has not read yet
        # two pinned buffers and events, used in turn: a launched step's tokens arrive in one while
        # the host still reads the other
        self._token_buffers = [torch.empty(max(max_batch_size, 1), dtype=torch.int32, pin_memory=True) for _ in range(2)] \
            if torch.cuda.is_available() else []
        self._token_events = [torch.cuda.Event() for _ in self._token_buffers]
        self._turn = 0

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

    def _entries(self, plan: StepPlan) -> List[StepEntry]:
        return [StepEntry(e.request.request_id, e.tokens, [len(e.tokens) - 1] if e.samples else []) for e in plan.entries]

    def _commit(self, plan: StepPlan, sampling: List[Request], tokens: Sequence[int],
                on_token: Optional[Callable[[Hashable, int], None]]) -> List[Request]:
        sampled = {r.request_id: int(t) for r, t in zip(sampling, tokens)}
        before = {r.request_id: len(r.output) for r in sampling}
        done = self.scheduler.commit(plan, sampled)
        if on_token is not None:
            for r in sampling:
                if len(r.output) > before[r.request_id]:
                    on_token(r.request_id, r.output[-1])
        return done

    def _checked(self, status, *plans) -> None:
        """Before a step's samples are committed: did one of its kernels give up a bounded wait? Then
        its samples, and those of a step launched on top of them, mean nothing: the requests of
        ``plans`` are aborted (pages and slots go back), nothing is committed, and the error is raised."""
        if status is None:
            return
        try:
            status.resolve(wait=True)
        except Exception:
            plans = [p for p in plans if p is not None]
            for plan in plans:
                for e in plan.entries:
                    self.scheduler.abort(e.request.request_id)
            for plan in plans:           # oldest first; every entry is void by now, nothing is appended
                self.scheduler.commit(plan, {})
            raise

    def _read(self, launched: _Launched, on_token, later: Optional[_Launched] = None) -> List[Request]:
        """The host catches up with a launched step: waits for its sampled tokens and commits them.
        ``later``: the step launched after it, which took its samples on the device."""
        launched.copied.synchronize()            # the status word was copied before the tokens
        self._checked(launched.status, launched.plan, later.plan if later is not None else None)
        return self._commit(launched.plan, launched.sampling, launched.tokens_host.tolist(), on_token)

    def step(self, on_token: Optional[Callable[[Hashable, int], None]] = None) -> List[Request]:
        """One scheduler iteration: plan, run the batch, sample, finish. Returns finished requests
        (with ``lookahead``: those of the step before the one launched now)."""
        previous = self._launched
        self._launched = None
        plan = self.scheduler.plan() if self.scheduler.has_work() else StepPlan()
        if not plan.entries:
            done = self._read(previous, on_token) if previous is not None else []
            if previous is None and not plan.preempted and self.scheduler.has_work():
                raise RuntimeError("scheduler stalled: no request can take a step with the pages that are free")
            return done
        feedback = (previous.tokens_dev, previous.row_of) if previous is not None else None
        # the logits are sampled from (on this stream, or read back) before the next step is launched
        logits = self.engine.step(self._entries(plan), feedback=feedback, borrow=True)
        status = self.engine.take_status()
        sampling = [e.request for e in plan.entries if e.samples]
        done: List[Request] = []
        launched = None
        if sampling and self.lookahead:
            tokens_dev = sample_on_device(logits, [r.params for r in sampling], [r.rng for r in sampling])
            if tokens_dev is not None:
                self._turn ^= 1
                launched = _Launched(plan, sampling, tokens_dev, self._token_buffers[self._turn], self._token_events[self._turn],
                                     status)
        if previous is not None:                       # the step before: its tokens have had a whole step to arrive
            done += self._read(previous, on_token, launched if launched is not None else _Unread(plan))
        if launched is None:                           # read this step's samples now (ranked rows, or no lookahead)
            tokens = sample(logits, [r.params for r in sampling], [r.rng for r in sampling]) if sampling else []
            self._checked(status, plan)
            done += self._commit(plan, sampling, tokens, on_token)
        self._launched = launched
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

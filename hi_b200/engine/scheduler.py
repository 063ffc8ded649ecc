"""The scheduler above the step function: admit, cut prompts into portions under a token
budget, decode, finish and free. Host-only; it decides, the engine runs.

Compared with the reference's continuous loop (crates/hi-cuda/src/lib.rs:4418-4471,
5062-5298): that one leases all pages of a request at admission and runs prefill chunks and
decode rows as separate forwards; this one takes pages step by step and puts decode tokens
and prompt portions into ONE batch.

When pages run out, in this order:
  1. no new request is admitted;
  2. prompt portions are shrunk to the pages that are free, or wait a step;
  3. if a DECODE token cannot get its page, the most recently admitted running request is
     preempted: its pages and slot go back, and it returns to the head of the waiting queue
     with prompt + generated tokens as its prompt and its generator state kept;
  4. a request that could never fit is refused when it is added (``insufficient_gpu_memory``,
     crates/hi-cuda/src/lib.rs:845-858).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, Hashable, List, Optional, Sequence, Tuple

from ..cache.pages import CacheManager
from ..sampling.sampler import DEFAULT_SEED, Lcg, SamplingParams

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


@dataclass
class SchedulerConfig:
    """Names as the reference's flags (crates/hi-local/src/main.rs:28-59,
    crates/hi-cuda/src/lib.rs:426-435)."""

    max_batch_size: int = 8              # requests in one step
    max_active_requests: Optional[int] = None   # running at a time; default = max_batch_size
    max_batched_tokens: int = 8192       # token budget of one step
    max_prefill_portion: Optional[int] = None   # longest prompt portion in one step

    def validate(self) -> None:
        if self.max_batch_size < 1 or self.max_batched_tokens < 1:
            raise ValueError("max_batch_size and max_batched_tokens must be positive")
        if self.max_active_requests is not None and self.max_active_requests < 1:
            raise ValueError("max_active_requests must be positive")
        if self.max_prefill_portion is not None and self.max_prefill_portion < 1:
            raise ValueError("max_prefill_portion must be positive")


@dataclass(eq=False)          # requests are compared by identity
class Request:
    request_id: Hashable
    prompt: List[int]
    params: SamplingParams
    output: List[int] = field(default_factory=list)
    status: str = WAITING
    finish_reason: Optional[str] = None
    computed: int = 0                    # tokens whose keys are in the cache
    preemptions: int = 0
    rng: Lcg = None                      # type: ignore[assignment]

    def __post_init__(self):
        if self.rng is None:
            self.rng = Lcg(DEFAULT_SEED if self.params.seed is None else self.params.seed)

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def pending(self) -> int:
        return len(self.prompt) + len(self.output) - self.computed

    @property
    def last_token(self) -> int:
        return self.output[-1] if self.output else self.prompt[-1]

    def span(self, begin: int, end: int) -> List[int]:
        """Tokens ``begin .. end`` of prompt + output, without building the whole list."""
        n = len(self.prompt)
        if end <= n:
            return self.prompt[begin:end]
        if begin >= n:
            return self.output[begin - n:end - n]
        return self.prompt[begin:] + self.output[:end - n]


@dataclass
class PlannedEntry:
    request: Request
    tokens: List[int]
    samples: bool          # the portion ends at the request's last token: its logits are wanted


@dataclass
class StepPlan:
    entries: List[PlannedEntry] = field(default_factory=list)
    preempted: List[Request] = field(default_factory=list)

    @property
    def n_tokens(self) -> int:
        return sum(len(e.tokens) for e in self.entries)


class Scheduler:
    def __init__(self, manager: CacheManager, config: SchedulerConfig, eos_token_ids: Sequence[int] = (),
                 max_model_len: Optional[int] = None, release: Optional[Callable[[Hashable], None]] = None):
        config.validate()
        self.manager, self.config = manager, config
        self.eos = set(int(t) for t in eos_token_ids)
        self.max_model_len = max_model_len
        self.release = release or (lambda rid: manager.close(rid) if manager.is_open(rid) else None)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []          # in admission order
        self.finished: List[Request] = []
        self.counters = {"admitted": 0, "preemptions": 0, "steps": 0, "shrunk_portions": 0, "stalled_portions": 0}

    # ------------------------------------------------------------------ admission
    @property
    def max_active(self) -> int:
        limit = self.config.max_active_requests or self.config.max_batch_size
        return min(limit, self.manager.max_requests)

    def add(self, request: Request) -> None:
        request.params.validate()
        if not request.prompt:
            raise ValueError("invalid_request_parameter: the prompt is empty")
        total = len(request.prompt) + request.params.max_tokens
        if self.max_model_len is not None and total > self.max_model_len:
            raise ValueError(f"context_length_exceeded: prompt ({len(request.prompt)}) + max_tokens "
                             f"({request.params.max_tokens}) exceeds the model's {self.max_model_len} positions")
        ps = self.manager.page_size
        for g, (spec, pool) in enumerate(zip(self.manager.groups, self.manager.pools)):
            if spec.window is None:
                need = -(-total // ps)
            else:
                # a windowed group holds at most its window plus the page being written
                need = min(-(-total // ps), -(-spec.window[1] // ps) + 1)
            if need > pool.total:
                raise ValueError(f"insufficient_gpu_memory: the request needs {need} page(s) of group {g}, "
                                 f"the pool has {pool.total}")
        request.status = WAITING
        self.waiting.append(request)

    def abort(self, request_id: Hashable) -> Optional[Request]:
        for r in list(self.running):
            if r.request_id == request_id:
                self.running.remove(r)
                self._finish(r, "aborted")
                return r
        for r in list(self.waiting):
            if r.request_id == request_id:
                self.waiting.remove(r)
                self._finish(r, "aborted")
                return r
        return None

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ planning
    def _fits(self, request: Request, n: int, promised: List[int], opened: bool) -> bool:
        need = self.manager.pages_needed(request.request_id if opened else None, n, request.computed)
        return all(promised[g] + need[g] <= self.manager.pools[g].free for g in range(len(need)))

    def _largest_fit(self, request: Request, n: int, promised: List[int], opened: bool) -> int:
        if self._fits(request, n, promised, opened):
            return n
        lo, hi = 0, n            # lo fits (0 tokens need nothing), hi does not
        while hi - lo > 1:
            mid = (lo + hi) // 2
            if self._fits(request, mid, promised, opened):
                lo = mid
            else:
                hi = mid
        return lo

    def _promise(self, request: Request, n: int, promised: List[int], opened: bool) -> None:
        need = self.manager.pages_needed(request.request_id if opened else None, n, request.computed)
        for g, v in enumerate(need):
            promised[g] += v

    def _preempt(self, victim: Request, plan: StepPlan) -> None:
        self.running.remove(victim)
        self.release(victim.request_id)
        victim.status = WAITING
        victim.computed = 0
        victim.preemptions += 1
        self.counters["preemptions"] += 1
        self.waiting.appendleft(victim)
        plan.preempted.append(victim)
        plan.entries = [e for e in plan.entries if e.request is not victim]

    def plan(self) -> StepPlan:
        """Decide the next step. Preemptions are carried out (through ``release``) here."""
        cfg = self.config
        plan = StepPlan()
        budget = cfg.max_batched_tokens
        promised = [0] * len(self.manager.groups)

        # 1. every running request that has one token pending decodes, oldest first
        decoding = [r for r in self.running if r.pending == 1 and r.computed >= len(r.prompt)]
        planned = set()                        # ids of requests with an entry in this plan
        i = 0
        while i < len(decoding) and budget > 0 and len(plan.entries) < cfg.max_batch_size:
            r = decoding[i]
            if r.status != RUNNING:             # preempted meanwhile
                i += 1
                continue
            if self._fits(r, 1, promised, True):
                self._promise(r, 1, promised, True)
                plan.entries.append(PlannedEntry(r, [r.last_token], True))
                planned.add(id(r))
                budget -= 1
                i += 1
                continue
            victim = self.running[-1]
            if victim is r and len(self.running) == 1:
                self.running.remove(r)
                self._finish(r, "insufficient_gpu_memory")
                i += 1
                continue
            # the victim's promised pages, if it was planned, come back with it
            if id(victim) in planned:
                planned.discard(id(victim))
                promised = [0] * len(self.manager.groups)
                self._preempt(victim, plan)
                budget = cfg.max_batched_tokens
                for e in plan.entries:
                    self._promise(e.request, len(e.tokens), promised, True)
                    budget -= len(e.tokens)
            else:
                self._preempt(victim, plan)
            # try r again (unless it was the victim)

        # 2. running requests still in their prompt get portions, oldest first
        for r in self.running:
            if budget <= 0 or len(plan.entries) >= cfg.max_batch_size:
                break
            if id(r) in planned or r.pending <= 0:
                continue
            self._plan_portion(r, plan, promised, budget, opened=True)
            budget = cfg.max_batched_tokens - plan.n_tokens

        # 3. admit waiting requests into what is left
        if not plan.preempted:
            slots_left = self.manager.free_slots
            while (self.waiting and budget > 0 and len(plan.entries) < cfg.max_batch_size
                   and len(self.running) < self.max_active and slots_left > 0):
                r = self.waiting[0]
                before = len(plan.entries)
                self._plan_portion(r, plan, promised, budget, opened=False)
                if len(plan.entries) == before:
                    break                       # no page for even one token: wait
                self.waiting.popleft()
                r.status = RUNNING
                self.running.append(r)
                self.counters["admitted"] += 1
                slots_left -= 1
                budget = cfg.max_batched_tokens - plan.n_tokens
        self.counters["steps"] += 1
        return plan

    def _plan_portion(self, r: Request, plan: StepPlan, promised: List[int], budget: int, opened: bool) -> None:
        want = min(r.pending, budget)
        if self.config.max_prefill_portion is not None:
            want = min(want, self.config.max_prefill_portion)
        n = self._largest_fit(r, want, promised, opened)
        if n <= 0:
            self.counters["stalled_portions"] += 1
            return
        if n < want:
            self.counters["shrunk_portions"] += 1
        self._promise(r, n, promised, opened)
        toks = r.span(r.computed, r.computed + n)
        plan.entries.append(PlannedEntry(r, toks, samples=(r.computed + n == len(r.prompt) + len(r.output))))

    # ------------------------------------------------------------------ after the step
    def commit(self, plan: StepPlan, sampled: Dict[Hashable, int]) -> List[Request]:
        """The step ran; ``sampled`` holds one token for every entry with ``samples``.
        Returns the requests that finished (their cache is released here)."""
        done: List[Request] = []
        for e in plan.entries:
            r = e.request
            r.computed += len(e.tokens)
            if not e.samples:
                continue
            tok = int(sampled[r.request_id])
            is_eos = (tok in self.eos and not r.params.ignore_eos) or tok in r.params.stop_token_ids
            if is_eos:
                reason = "stop"                 # EOS is not emitted (crates/hi-mlx/src/models.rs:598-600)
            else:
                r.output.append(tok)
                reason = "length" if len(r.output) >= r.params.max_tokens else None
            if reason:
                self.running.remove(r)
                self._finish(r, reason)
                done.append(r)
        return done

    def _finish(self, r: Request, reason: str) -> None:
        r.status, r.finish_reason = FINISHED, reason
        self.release(r.request_id)
        self.finished.append(r)

"""The scheduler above the step function: admit, cut prompts into portions under a token
budget, decode, finish and free. Host-only; it decides, the engine runs. The decisions are
taken by the native host runtime (``hi_b200/csrc/host/scheduler.cpp``), which works on counts;
this module is its Python face and keeps what only the caller knows: token values, sampling
parameters, generator state, end-of-sequence ids.

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

import ctypes
from dataclasses import dataclass, field
from typing import Callable, Dict, Hashable, List, Optional, Sequence

from ..cache.pages import CacheManager
from ..host import build as host
from ..sampling.sampler import DEFAULT_SEED, Lcg, SamplingParams

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"
IN_FLIGHT = -1     # in a planned entry's tokens: the token that the step before samples (its value is on the device)
_STATUS = {0: WAITING, 1: RUNNING, 2: FINISHED}
_REASON = {0: None, 1: "length", 2: "stop", 3: "aborted", 4: "insufficient_gpu_memory"}


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


class Request:
    """One generation request. ``status``, ``computed`` (tokens whose keys are in the cache) and
    ``preemptions`` are the scheduler's; they are read from it while it knows the request."""

    def __init__(self, request_id: Hashable, prompt: List[int], params: SamplingParams,
                 output: Optional[List[int]] = None, rng: Optional[Lcg] = None):
        self.request_id, self.prompt, self.params = request_id, prompt, params
        self.output: List[int] = [] if output is None else output
        self.finish_reason: Optional[str] = None
        self.rng = rng if rng is not None else Lcg(DEFAULT_SEED if params.seed is None else params.seed)
        self._scheduler: Optional["Scheduler"] = None
        self._handle = -1
        self._last = (WAITING, 0, 0)       # status, computed, preemptions once the scheduler has let go

    def _stat(self, what: int) -> Optional[int]:
        s = self._scheduler
        return None if s is None else int(s._lib.hbh_sched_request_stat(s._ptr, self._handle, what))

    @property
    def status(self) -> str:
        v = self._stat(0)
        return self._last[0] if v is None else _STATUS[v]

    @property
    def computed(self) -> int:
        v = self._stat(1)
        return self._last[1] if v is None else v

    @property
    def preemptions(self) -> int:
        v = self._stat(2)
        return self._last[2] if v is None else v

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

    def __repr__(self) -> str:
        return f"Request({self.request_id!r}, prompt={len(self.prompt)}, output={len(self.output)}, {self.status})"


@dataclass
class PlannedEntry:
    request: Request
    tokens: List[int]      # the last one is IN_FLIGHT when the step before samples it
    samples: bool          # the portion ends at the request's last token: its logits are wanted


@dataclass
class StepPlan:
    entries: List[PlannedEntry] = field(default_factory=list)
    preempted: List[Request] = field(default_factory=list)
    plan_id: int = 0

    @property
    def n_tokens(self) -> int:
        return sum(len(e.tokens) for e in self.entries)


class _Counters:
    """``scheduler.counters``: read from the native scheduler."""

    _NAMES = ("admitted", "preemptions", "steps", "shrunk_portions", "stalled_portions")

    def __init__(self, scheduler: "Scheduler"):
        self._s = scheduler

    def __getitem__(self, name: str) -> int:
        return int(self._s._lib.hbh_sched_counter(self._s._ptr, self._NAMES.index(name)))

    def keys(self):
        return list(self._NAMES)

    def __iter__(self):
        return iter(self._NAMES)


class Scheduler:
    def __init__(self, manager: CacheManager, config: SchedulerConfig, eos_token_ids: Sequence[int] = (),
                 max_model_len: Optional[int] = None, release: Optional[Callable[[Hashable], None]] = None):
        config.validate()
        self.manager, self.config = manager, config
        self.eos = set(int(t) for t in eos_token_ids)
        self.max_model_len = max_model_len
        self._lib = host.library()
        self._ptr = self._lib.hbh_sched_create(manager._ptr, config.max_batch_size, config.max_active_requests or 0,
                                               config.max_batched_tokens, config.max_prefill_portion or 0,
                                               int(max_model_len or 0))
        if not self._ptr:
            raise ValueError("the native scheduler refused this configuration")
        self.release = release
        if release is not None:
            handles = manager._handles

            def call_release(_user, handle):
                release(handles.of_handle[handle])

            self._release_c = host.RELEASE_FN(call_release)      # kept alive with the scheduler
            self._lib.hbh_sched_set_release(self._ptr, self._release_c, None)
        self._live: Dict[int, Request] = {}          # handle -> request the native scheduler knows
        self.finished: List[Request] = []
        self.counters = _Counters(self)
        cap = max(config.max_batch_size, manager.max_requests, 1) + 1
        self._cap = cap
        self._entries = (ctypes.c_int64 * (5 * cap))()
        self._preempted = (ctypes.c_int64 * cap)()
        self._dropped = (ctypes.c_int64 * cap)()
        self._finished = (ctypes.c_int64 * (2 * cap))()
        self._counts = (ctypes.c_int * 3)()

    def __del__(self):
        if getattr(self, "_ptr", None):
            self._lib.hbh_sched_destroy(self._ptr)
            self._ptr = None

    # ------------------------------------------------------------------ admission
    @property
    def max_active(self) -> int:
        limit = self.config.max_active_requests or self.config.max_batch_size
        return min(limit, self.manager.max_requests)

    def _queue(self, which: int) -> List[Request]:
        n = self._lib.hbh_sched_queue(self._ptr, which, None, 0)
        buf = (ctypes.c_int64 * max(n, 1))()
        self._lib.hbh_sched_queue(self._ptr, which, buf, n)
        return [self._live[buf[i]] for i in range(n)]

    @property
    def waiting(self) -> List[Request]:
        return self._queue(0)

    @property
    def running(self) -> List[Request]:          # in admission order
        return self._queue(1)

    def add(self, request: Request) -> None:
        request.params.validate()
        if not request.prompt:
            raise ValueError("invalid_request_parameter: the prompt is empty")
        handles = self.manager._handles
        h = handles.pin(request.request_id)
        code = self._lib.hbh_sched_add(self._ptr, h, len(request.prompt), int(request.params.max_tokens))
        if code != host.OK:
            handles.unpin(h)
            handles.drop_if_unused(h, self.manager.is_open(request.request_id))
            if code in (host.ERR_CONTEXT_LENGTH, host.ERR_NEVER_FITS):
                raise ValueError(self._lib.hbh_sched_error(self._ptr).decode())
            if code == host.ERR_ALREADY_OPEN:
                raise ValueError(f"invalid_request_parameter: request {request.request_id!r} is already scheduled")
            raise ValueError(f"invalid_request_parameter: the scheduler refused the request (code {code})")
        request._scheduler, request._handle = self, h
        self._live[h] = request

    def _let_go(self, r: Request, reason: Optional[str]) -> None:
        """The request is finished: keep its last state on the Python object, drop the native record."""
        r._last = (FINISHED, r.computed, r.preemptions)
        if reason is not None:
            r.finish_reason = reason
        h = r._handle
        r._scheduler = None
        self._lib.hbh_sched_forget(self._ptr, h)
        self._live.pop(h, None)
        handles = self.manager._handles
        handles.unpin(h)
        handles.drop_if_unused(h, self.manager.is_open(r.request_id))
        self.finished.append(r)

    def abort(self, request_id: Hashable) -> Optional[Request]:
        h = self.manager._handles.get(request_id)
        r = self._live.get(h) if h is not None else None
        if r is None or not self._lib.hbh_sched_abort(self._ptr, h):
            return None
        self._let_go(r, "aborted")
        return r

    def assume_running(self, request: Request, computed: int) -> None:
        """Benchmarks only: a waiting request whose first ``computed`` tokens the caller has put
        into the cache by other means (``Engine.assume_cached``) starts running from there."""
        if self._lib.hbh_sched_assume_running(self._ptr, request._handle, int(computed)) != host.OK:
            raise ValueError(f"request {request.request_id!r} is not waiting, or {computed} is not inside its tokens")

    def has_work(self) -> bool:
        return bool(self._lib.hbh_sched_has_work(self._ptr))

    # ------------------------------------------------------------------ planning
    def plan(self) -> StepPlan:
        """Decide the next step. Preemptions are carried out (through ``release``) here. The plan
        counts as carried out at once; a second plan may be made before the first is committed
        (its entries then hold ``IN_FLIGHT`` where the first one's sample goes), not a third."""
        c = self._counts
        plan_id = ctypes.c_int64(0)
        code = self._lib.hbh_sched_plan(self._ptr, ctypes.byref(plan_id), self._entries, self._cap, ctypes.byref(c, 0),
                                        self._preempted, self._cap, ctypes.byref(c, 4), self._dropped, self._cap,
                                        ctypes.byref(c, 8))
        if code != host.OK:
            raise RuntimeError(f"the native scheduler failed to plan (code {code}): "
                               f"{self._lib.hbh_sched_error(self._ptr).decode()}")
        plan = StepPlan(plan_id=plan_id.value)
        for i in range(c[0]):
            h, begin, count, samples, in_flight = self._entries[5 * i: 5 * i + 5]
            r = self._live[h]
            toks = r.span(begin, begin + count - 1) + [IN_FLIGHT] if in_flight else r.span(begin, begin + count)
            plan.entries.append(PlannedEntry(r, toks, bool(samples)))
        plan.preempted = [self._live[self._preempted[i]] for i in range(c[1])]
        for i in range(c[2]):            # a lone decode that cannot get a page
            self._let_go(self._live[self._dropped[i]], "insufficient_gpu_memory")
        return plan

    # ------------------------------------------------------------------ after the step
    def commit(self, plan: StepPlan, sampled: Dict[Hashable, int]) -> List[Request]:
        """The step ran; ``sampled`` holds one token for every entry with ``samples``.
        Returns the requests that finished (their cache is released here)."""
        if not plan.entries:                # an empty plan was never outstanding
            return []
        stops, appended = [], []
        for e in plan.entries:
            if not e.samples:
                continue
            r = e.request
            if r._scheduler is None:        # it ended after this entry was planned: nobody reads the sample
                stops.append(0)
                continue
            tok = int(sampled[r.request_id])
            stop = (tok in self.eos and not r.params.ignore_eos) or tok in r.params.stop_token_ids
            if not stop:                    # EOS is not emitted (crates/hi-mlx/src/models.rs:598-600)
                appended.append((r, tok))
            stops.append(1 if stop else 0)
        n = ctypes.c_int(0)
        code = self._lib.hbh_sched_commit(self._ptr, plan.plan_id, (ctypes.c_int * max(len(stops), 1))(*stops), len(stops),
                                          self._finished, self._cap, ctypes.byref(n))
        if code != host.OK:
            raise RuntimeError(f"the native scheduler failed to commit (code {code}): "
                               f"{self._lib.hbh_sched_error(self._ptr).decode()}")
        for r, tok in appended:
            r.output.append(tok)
        done: List[Request] = []
        for i in range(n.value):
            r = self._live[self._finished[2 * i]]
            self._let_go(r, _REASON[self._finished[2 * i + 1]])
            done.append(r)
        return done

"""The engine: a model on one GPU, its cache, and the ONE step function.

``Engine.step`` takes a batch of (request, its next tokens): portions of prompts beside
single decoded tokens, cut anywhere. It runs only those tokens, as one batch, against the
cache that earlier steps left, and returns float32 logits at the wanted places. The
scheduler, ``generate`` and the trace replay all drive this same function. (The reference
has three separate forwards for whole prompts, one span, and decode rows:
crates/hi-cuda/src/gpu.rs:8842-8929, 10541-10715, 9026-9132.)
"""
from __future__ import annotations

import gc
import itertools
import os
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.device import DeviceCache, plan_groups, pool_tokens_for_budget
from ..cache.pages import CacheManager, OutOfPages
from ..config.registry import load_architecture, lookup
from ..parts.context import StepContext
from ..parts.linear import configure_matmul_precision
from ..parts.model import Model
from ..kernels import ops
from ..weights.loader import load_from_dir, load_random

IN_FLIGHT = -1     # a token that the step before samples: its value is on the device, not on the host

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           "f32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name in (torch.bfloat16, torch.float32):
            return name
    elif str(name).lower() in _DTYPES:
        return _DTYPES[str(name).lower()]
    raise ValueError(f"dtype {name!r} is not supported (bfloat16 or float32)")


def _require_cuda(device) -> None:
    if not torch.cuda.is_available() or torch.device(device).type != "cuda":
        raise RuntimeError("hi_b200 needs a CUDA device; there is no CPU path")
    configure_matmul_precision()


def _check_kernel_status(force: bool = False) -> None:
    """A tensor-core kernel that gave up a bounded wait makes the step fail loudly."""
    if ops.TC_USED[0] or force:
        ops.check_tc_status()


def _count_launches(n: int) -> None:
    ops.LAUNCHES[0] += n


def _pinned_int32(n: int) -> torch.Tensor:
    return torch.empty(n, dtype=torch.int32, pin_memory=True)


@dataclass
class StepEntry:
    """The next tokens of one request in one step; ``want`` indexes into ``tokens``."""

    request_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class EngineStats:
    steps: int = 0
    tokens: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    logit_rows: int = 0


class Engine:
    """One model on one CUDA device.

    ``kv_cache_tokens`` sizes every page pool (tokens, rounded up to pages);
    ``windowed_cache_tokens`` optionally gives the windowed groups (chunked layers) a smaller
    pool. Without ``kv_cache_tokens`` the pools are sized from the device memory that is free once
    the weights are loaded: ``cache_memory_fraction`` of it, windowed groups at what
    ``max_active_requests`` windows need, the rest to the groups that keep every key.
    ``max_active_requests`` is the number of state slots / block-table rows.
    """

    def __init__(self, model: Model, *, kv_page_size: int = 64, kv_cache_tokens: Optional[int] = None,
                 windowed_cache_tokens: Optional[int] = None, max_active_requests: int = 8,
                 cache_memory_fraction: float = 0.9,
                 debug_poison: bool = False, use_cuda_graphs: bool = True, graph_context_bucket: int = 1024,
                 max_graphs: int = 16):
        _require_cuda(model.device)
        self.model = model
        self.device = model.device
        self.dtype = model.dtype
        self.page_size = int(kv_page_size)
        groups, self.group_of = plan_groups(model.cache_specs)
        auto = None
        if kv_cache_tokens is None:
            if not 0.0 < cache_memory_fraction <= 1.0:
                raise ValueError("cache_memory_fraction must lie in (0, 1]")
            free, _total = torch.cuda.mem_get_info(self.device)
            longest = model.spec.max_position_embeddings
            auto = pool_tokens_for_budget(model.cache_specs, torch.empty((), dtype=model.dtype).element_size(),
                                          int(free * cache_memory_fraction), self.page_size, max_active_requests,
                                          most_tokens=None if longest is None else longest * max_active_requests)
        pages = []
        for g, spec in enumerate(groups):
            if auto is not None:
                tokens = auto[g] if (spec.window is None or windowed_cache_tokens is None) else windowed_cache_tokens
            else:
                tokens = kv_cache_tokens if (spec.window is None or windowed_cache_tokens is None) else windowed_cache_tokens
            pages.append(max(1, -(-int(tokens) // self.page_size)))
        self.manager = CacheManager(groups, pages, self.page_size, max_active_requests)
        self.cache = DeviceCache(model.cache_specs, pages, self.page_size, max_active_requests, model.dtype,
                                 self.device)
        self.vocab_size = model.spec.vocab_size
        self.stats = EngineStats()
        self.debug_poison = debug_poison
        self.use_cuda_graphs = use_cuda_graphs and model.graph_safe
        self._graphs: Dict[Tuple[int, int], "_DecodeGraph"] = {}
        if graph_context_bucket < 1 or max_graphs < 1:
            raise ValueError("graph_context_bucket and max_graphs must be positive")
        # a captured decode step serves contexts up to a multiple of this many tokens
        self.context_bucket = -(-int(graph_context_bucket) // self.page_size) * self.page_size
        self.max_graphs = int(max_graphs)
        self.last_step_h2d_bytes = 0
        # captured steps whose kernels wait with a limit: their status word follows them to pinned
        # memory (four tickets used in turn) and is read later, by whoever uses the step's result
        self._status_ring: List[ops.PendingStatus] = []
        self._status_turn = 0
        self.last_status: Optional[ops.PendingStatus] = None    # the ticket of the step run last (None: checked already)

    # ------------------------------------------------------------------ construction
    @staticmethod
    def from_dir(model_dir: str, dtype="bfloat16", device="cuda:0", **options) -> "Engine":
        """Load a model folder (config.json + safetensors); the model class is chosen by config.json."""
        arch, cfg, _raw = load_architecture(model_dir)
        model = Model(arch.build_spec(cfg), parse_dtype(dtype), device)
        load_from_dir(model, model_dir, arch.normalize_tensor_name, arch.derive_tensors)
        return Engine(model, **options)

    @staticmethod
    def from_config(config: dict, seed: int = 0, std: float = 0.02, dtype="bfloat16", device="cuda:0",
                    **options) -> "Engine":
        """Random weights generated on the device from ``seed`` (no files): for large benchmarks."""
        arch = lookup(config)
        model = Model(arch.build_spec(arch.parse_config(config, None)), parse_dtype(dtype), device)
        load_random(model, seed, std)
        return Engine(model, **options)

    # ------------------------------------------------------------------ requests
    def open(self, request_id: Hashable) -> None:
        slot = self.manager.open(request_id)
        self.cache.reset_slot(slot)

    def finish(self, request_id: Hashable) -> None:
        """The request is over: its pages and its slot go back."""
        if self.manager.is_open(request_id):
            self.manager.close(request_id)

    def length(self, request_id: Hashable) -> int:
        return self.manager.length(request_id) if self.manager.is_open(request_id) else 0

    def assume_cached(self, request_id: Hashable, length: int) -> None:
        """Benchmarks only: treat ``length`` tokens of a new request as already in the cache
        (pages are taken; their contents are whatever the pools hold). Lets a decode step at a
        long context be timed without running the prefill that would produce it."""
        self.open(request_id)
        done = 0
        while done < length:          # in runs, so that windowed groups never hold more than a window
            n = min(4096, length - done)
            self.manager.reserve(request_id, n)
            self.manager.commit(request_id, n)
            done += n

    # ------------------------------------------------------------------ the step
    def step(self, entries: Sequence[StepEntry], tap=None, feedback=None, borrow: bool = False,
             forced=None) -> Optional[torch.Tensor]:
        """Run one batch. Returns float32 logits [wanted, vocab] on the device, in the order
        of the entries and of each entry's ``want`` (None if nothing is wanted). ``tap(name,
        tensor)``, if given, is called by parts that report intermediate tensors (router ids),
        in the step's flat token order (crates/hi-cuda/src/lib.rs:87-201 has such a dump hook).

        ``feedback = (sampled, rows)``: an entry whose last token is ``IN_FLIGHT`` (-1) takes it on
        the device from ``sampled[rows[request_id]]``, an int32 tensor that the step before this
        one filled (its sampled tokens): the step can be launched before the host has read them.

        ``borrow``: the caller uses the logits before it runs the next step (work queued on this
        stream counts), so a captured step may hand out its own output buffer instead of a copy."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        self._resolve_status(wait=False)
        if not entries:
            return None
        fed = feedback[1] if feedback is not None else {}
        seen = set()
        for e in entries:
            if e.request_id in seen:
                raise ValueError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            if len(e.tokens) == 0:
                raise ValueError(f"request {e.request_id!r} brings no tokens")
            known = e.tokens[:-1] if (e.tokens[-1] == IN_FLIGHT and e.request_id in fed) else e.tokens
            bad = [t for t in known if not 0 <= int(t) < self.vocab_size]
            if bad:
                raise ValueError(f"request {e.request_id!r}: token ids {bad[:4]} outside 0..{self.vocab_size - 1}")
            if any(not 0 <= int(w) < len(e.tokens) for w in e.want):
                raise ValueError(f"request {e.request_id!r}: 'want' {list(e.want)} outside its {len(e.tokens)} tokens")
        # pages for every entry, or for none
        opened, reserved = [], []
        try:
            for e in entries:
                if not self.manager.is_open(e.request_id):
                    self.open(e.request_id)
                    opened.append(e.request_id)
                reserved.append((e.request_id, self.manager.table_lengths(e.request_id)))
                self.manager.reserve(e.request_id, len(e.tokens))
        except Exception:
            for rid, before in reserved:
                if rid not in opened:
                    self.manager.unreserve(rid, before)
            for rid in opened:
                self.manager.close(rid)
            raise

        self.last_status = None
        graph = self._decode_graph_for(entries, feedback) if forced is None else None
        if graph is not None:
            self._build_context(entries, widths=graph.widths, static=graph, feedback=feedback)
            graph.graph.replay()
            _count_launches(graph.kernels)
            if tap is not None:                  # what the parts reported at capture sits in the graph's own
                for name, tensor in graph.taps.items():     # buffers, refilled by every replay
                    tap(name, tensor)
            if graph.uses_tensor_core_experts:
                # no sync here: the status word follows the kernels to pinned memory; a caller that
                # commits the step's result resolves `last_status` first, and whatever is still
                # open is read at the start of a later step or when the engine is asked for its state
                if not self._status_ring:
                    self._status_ring = [ops.PendingStatus(self.device) for _ in range(4)]
                ticket = self._status_ring[self._status_turn % len(self._status_ring)]
                self._status_turn += 1
                ticket.enqueue()
                ticket.claimed = False
                self.last_status = ticket
            logits = graph.logits if borrow else graph.logits.clone()
            ctx, logit_rows = graph.ctx, graph.logit_rows
        else:
            ctx, logit_rows = self._build_context(entries, feedback=feedback)
            ctx.tap, ctx.forced = tap, forced
            logits = self.model.forward(ctx, self.cache.views, logit_rows)
            _check_kernel_status()
        for e in entries:
            returned = self.manager.commit(e.request_id, len(e.tokens))
            if self.debug_poison and returned:
                self.cache.poison_pages(returned)
        st = self.stats
        st.steps += 1
        st.tokens += ctx.n_tokens
        for e in entries:
            if len(e.tokens) == 1:
                st.decode_tokens += 1
            else:
                st.prefill_tokens += len(e.tokens)
        st.logit_rows += 0 if logit_rows is None else int(logit_rows.numel())
        return logits

    def _build_context(self, entries: Sequence[StepEntry], widths: Optional[List[int]] = None,
                       static: Optional["_DecodeGraph"] = None, feedback=None
                       ) -> Tuple[StepContext, Optional[torch.Tensor]]:
        """All of a step's integer inputs in one pinned buffer, one host-to-device copy.
        With ``static`` the buffers of a captured decode graph are filled instead."""
        mgr = self.manager
        n_seqs = len(entries)
        n_new = [len(e.tokens) for e in entries]
        n_tokens = sum(n_new)
        handles = mgr.handles_of([e.request_id for e in entries])
        if widths is None:
            widths = mgr.step_widths(handles)
        n_want = sum(len(e.want) for e in entries)
        # tokens that the step before this one sampled and the host has not read: (place, row) pairs
        fed_dst, fed_src, cursor = [], [], 0
        for e in entries:
            cursor += len(e.tokens)
            if feedback is not None and e.tokens[-1] == IN_FLIGHT:
                fed_dst.append(cursor - 1)
                fed_src.append(feedback[1][e.request_id])
        n_fed = len(fed_dst)
        fed_room = n_seqs if static is not None else n_fed

        def pad4(n):
            return (n + 3) // 4 * 4

        sizes = [n_tokens, n_tokens, n_tokens, n_seqs + 1, n_seqs, n_want] + [n_seqs * w for w in widths] + \
            [fed_room, fed_room]
        offsets, total = [], 0
        for s in sizes:
            offsets.append(total)
            total += pad4(s)
        if static is not None:
            static.copied.synchronize()          # the previous step's copy has left the pinned buffer
            host = static.host
        else:
            host = _pinned_int32(max(total, 4))
        o_tok, o_pos, o_seq, o_cu, o_slot, o_want = offsets[:6]
        # the native runtime fills the buffer: tokens, positions, sequence ids, cumulative counts,
        # slots, wanted rows and the block tables. A captured decode step keeps its table rows
        # between steps: a row is rewritten only when another request sits in it or the request's
        # tables changed (a new page, a freed chunk)
        if n_tokens == n_seqs:
            tokens = np.fromiter((e.tokens[0] for e in entries), dtype=np.int32, count=n_seqs)
        else:
            tokens = np.fromiter(itertools.chain.from_iterable(e.tokens for e in entries), dtype=np.int32, count=n_tokens)
        want_counts = np.fromiter((len(e.want) for e in entries), dtype=np.int32, count=n_seqs)
        want = np.fromiter(itertools.chain.from_iterable(e.want for e in entries), dtype=np.int32, count=n_want)
        n_new_a = np.asarray(n_new, dtype=np.int32)
        widths_a = np.asarray(widths if widths else [0], dtype=np.int32)
        offsets_a = np.asarray(offsets, dtype=np.int64)
        starts_a, slots_a = np.empty(n_seqs, dtype=np.int32), np.empty(n_seqs, dtype=np.int32)
        code = mgr._lib.hbh_pack_step(
            mgr._ptr, n_seqs, handles.ctypes.data, n_new_a.ctypes.data, tokens.ctypes.data, want_counts.ctypes.data,
            want.ctypes.data, widths_a.ctypes.data, offsets_a.ctypes.data, host.data_ptr(), starts_a.ctypes.data,
            slots_a.ctypes.data, static.row_request.ctypes.data if static is not None else None,
            static.row_version.ctypes.data if static is not None else None)
        if code != 0:
            raise RuntimeError(f"packing the step's inputs failed (code {code})")
        starts, slots = starts_a.tolist(), slots_a.tolist()
        o_fed_dst, o_fed_src = offsets[-2], offsets[-1]
        if n_fed:
            view = host.numpy()
            view[o_fed_dst: o_fed_dst + n_fed] = fed_dst
            view[o_fed_src: o_fed_src + n_fed] = fed_src
        self.last_step_h2d_bytes = host.numel() * 4     # the one host-to-device copy of this step
        if static is not None:
            static.dev.copy_(host, non_blocking=True)
            static.copied.record()
            if n_fed:
                ops.feed_tokens(static.ctx.tokens, static.dev[o_fed_dst: o_fed_dst + n_fed],
                                static.dev[o_fed_src: o_fed_src + n_fed], feedback[0])
            return static.ctx, static.logit_rows
        dev = host.to(self.device, non_blocking=True)
        if n_fed:
            ops.feed_tokens(dev[o_tok: o_tok + n_tokens], dev[o_fed_dst: o_fed_dst + n_fed],
                            dev[o_fed_src: o_fed_src + n_fed], feedback[0])

        def seg(off, n):
            return dev[off: off + n]

        block_tables = {g: seg(offsets[6 + g], n_seqs * widths[g]).view(n_seqs, widths[g])
                        for g in range(len(widths))}
        ctx = StepContext(
            n_tokens=n_tokens, n_seqs=n_seqs, tokens=seg(o_tok, n_tokens), positions=seg(o_pos, n_tokens),
            seq_of_token=seg(o_seq, n_tokens), cu_seqlens=seg(o_cu, n_seqs + 1), slots=seg(o_slot, n_seqs),
            start_pos=starts, n_new=n_new, slot_ids=slots, block_tables=block_tables, page_size=self.page_size,
            max_context=max(s + n for s, n in zip(starts, n_new)))
        ctx._host_buffer = host       # keep the pinned buffer alive until the copy has run
        singles = [s for s, n in enumerate(n_new) if n == 1]
        if singles and len(singles) < n_seqs:
            # rows of cu_seqlens for the single-token requests, picked on the device (no second copy)
            idx = torch.tensor(singles, dtype=torch.int64).to(self.device, non_blocking=True)
            ctx.decode_rows = ctx.cu_seqlens.index_select(0, idx).to(torch.int64)
            ctx.decode_max_context = max(starts[s] + 1 for s in singles)
        logit_rows = seg(o_want, n_want) if n_want else None
        return ctx, logit_rows

    # ------------------------------------------------------------------ captured decode steps
    def _decode_graph_for(self, entries: Sequence[StepEntry], feedback=None) -> Optional["_DecodeGraph"]:
        """A CUDA graph of the whole step for batches of single decoded tokens that all want
        their logits: same kernels as the eager step, launched once. Keyed by batch size and the
        context bucket (which fixes the block-table widths and the attention splits)."""
        if not self.use_cuda_graphs or any(len(e.tokens) != 1 or list(e.want) != [0] for e in entries):
            return None
        longest = max(self.manager.length(e.request_id) for e in entries) + 1
        bucket = -(-longest // self.context_bucket) * self.context_bucket
        key = (len(entries), bucket)
        graph = self._graphs.get(key)
        if graph is None:
            if len(self._graphs) >= self.max_graphs:          # the one captured longest ago makes room
                self._graphs.pop(next(iter(self._graphs)))
            graph = _DecodeGraph(self, len(entries), bucket)
            self._graphs[key] = graph
        if not graph.captured:
            if graph.eager_runs < 1:          # the first step of a shape runs eagerly (library warm-up)
                graph.eager_runs += 1
                return None
            graph.capture(entries, feedback)
        return graph

    def _resolve_status(self, wait: bool = True) -> None:
        """Read the status words that followed captured steps' kernels; without ``wait`` only those
        whose copy has run already (the next look, or ``snapshot``, catches up)."""
        for ticket in self._status_ring:
            if ticket.pending and not ticket.claimed:
                ticket.resolve(wait)

    def take_status(self) -> Optional[ops.PendingStatus]:
        """The status ticket of the step run last, for a caller that resolves it itself before it
        uses the step's result (the engine then leaves it alone). None: that step was checked when it ran."""
        ticket = self.last_status
        if ticket is not None:
            ticket.claimed = True
        return ticket

    # ------------------------------------------------------------------ bookkeeping
    def snapshot(self) -> dict:
        self._resolve_status()
        s = self.manager.snapshot()
        s.update(steps=self.stats.steps, tokens=self.stats.tokens, prefill_tokens=self.stats.prefill_tokens,
                 decode_tokens=self.stats.decode_tokens, cache_bytes=self.cache.bytes)
        return s


class _DecodeGraph:
    """Static buffers and the captured graph of one decode-step shape."""

    def __init__(self, engine: Engine, n_seqs: int, bucket: int):
        self.engine, self.n_seqs, self.bucket = engine, n_seqs, bucket
        self.widths = [-(-bucket // engine.page_size) for _ in engine.manager.groups]
        pad4 = lambda n: (n + 3) // 4 * 4
        sizes = [n_seqs, n_seqs, n_seqs, n_seqs + 1, n_seqs, n_seqs] + [n_seqs * w for w in self.widths] + \
            [n_seqs, n_seqs]                     # the last two: places and rows of tokens fed on the device
        offsets, total = [], 0
        for sz in sizes:
            offsets.append(total)
            total += pad4(sz)
        self.host = _pinned_int32(total)
        self.dev = torch.zeros(total, dtype=torch.int32, device=engine.device)
        self.copied = torch.cuda.Event()
        self.copied.record()
        seg = lambda off, n: self.dev[off: off + n]
        tables = {g: seg(offsets[6 + g], n_seqs * w).view(n_seqs, w) for g, w in enumerate(self.widths)}
        self.ctx = StepContext(
            n_tokens=n_seqs, n_seqs=n_seqs, tokens=seg(offsets[0], n_seqs), positions=seg(offsets[1], n_seqs),
            seq_of_token=seg(offsets[2], n_seqs), cu_seqlens=seg(offsets[3], n_seqs + 1), slots=seg(offsets[4], n_seqs),
            start_pos=[0] * n_seqs, n_new=[1] * n_seqs, slot_ids=[0] * n_seqs, block_tables=tables,
            page_size=engine.page_size, max_context=bucket)
        self.logit_rows = seg(offsets[5], n_seqs)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.captured = False
        self.eager_runs = 0
        self.row_request = np.full(n_seqs, -1, dtype=np.int64)    # request and table version last written
        self.row_version = np.full(n_seqs, -1, dtype=np.int64)    # into each table row
        self.kernels = 0
        self.uses_tensor_core_experts = False
        self.taps: Dict[str, torch.Tensor] = {}     # what parts reported while the step was captured

    def capture(self, entries: Sequence[StepEntry], feedback=None) -> None:
        eng = self.engine
        # valid inputs for the capture run: the tokens fed on the device included
        eng._build_context(entries, widths=self.widths, static=self, feedback=feedback)
        torch.cuda.synchronize()
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):                                   # once outside capture, on a side stream
            eng.model.forward(self.ctx, eng.cache.views, self.logit_rows)
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize()
        before = ops.LAUNCHES[0]
        ops.TC_USED[0] = False
        self.graph = torch.cuda.CUDAGraph()
        self.taps = {}
        self.ctx.tap = self.taps.__setitem__
        # Python's cycle collector must not run inside the capture: an engine dropped earlier and its
        # captured steps refer to each other, so the collector is what frees them, and freeing a CUDA
        # graph while a stream is being captured invalidates the capture. Collect now, then hold it off.
        gc.collect()
        collecting = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(self.graph):
                self.logits = eng.model.forward(self.ctx, eng.cache.views, self.logit_rows)
        finally:
            if collecting:
                gc.enable()
            self.ctx.tap = None
        self.kernels = ops.LAUNCHES[0] - before      # this library's kernels in one replay
        self.uses_tensor_core_experts = ops.TC_USED[0]
        ops.TC_USED[0] = False
        self.captured = True

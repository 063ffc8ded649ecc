"""Host side of the cache: pages, block tables, state slots. Pure Python, no device.

Layer groups with different needs (every earlier key, or a window of them) have pools of
their own; a request has one block table per group, indexed by ``position // page_size``.
Pages go back to their pool when the request ends or when the window has passed them, and
are handed out again (the reference allocates everything at admission and frees only at
retirement: crates/hi-cuda/src/lib.rs:641-957, 4781-4844).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

from ..parts.spec import CacheSpec

FREED = -1   # a block whose page was given back (the window has passed it)


class OutOfPages(RuntimeError):
    """insufficient_gpu_memory in the reference's terms (crates/hi-cuda/src/lib.rs:845-858)."""

    def __init__(self, group: int, needed: int, free: int, total: int):
        super().__init__(f"insufficient_gpu_memory: page group {group} needs {needed} page(s), "
                         f"only {free} of {total} free")
        self.group, self.needed, self.free, self.total = group, needed, free, total


class OutOfSlots(RuntimeError):
    pass


class PagePool:
    """Free list of one group. Every page has at most one owner; giving back a page that is
    not held, or not held by that owner, raises."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.total = num_pages
        self._free = deque(range(num_pages))
        self._owner: List[Optional[Hashable]] = [None] * num_pages
        self.peak_used = 0
        self.allocations = 0
        self.failed_allocations = 0

    @property
    def free(self) -> int:
        return len(self._free)

    @property
    def used(self) -> int:
        return self.total - len(self._free)

    def take(self, owner: Hashable) -> int:
        if not self._free:
            self.failed_allocations += 1
            raise OutOfPages(-1, 1, 0, self.total)
        page = self._free.popleft()
        assert self._owner[page] is None, f"page {page} handed out twice"
        self._owner[page] = owner
        self.allocations += 1
        self.peak_used = max(self.peak_used, self.used)
        return page

    def give(self, page: int, owner: Hashable) -> None:
        if not 0 <= page < self.total:
            raise ValueError(f"page {page} is outside the pool")
        if self._owner[page] is None:
            raise RuntimeError(f"page {page} freed twice")
        if self._owner[page] != owner:
            raise RuntimeError(f"page {page} is held by {self._owner[page]!r}, not by {owner!r}")
        self._owner[page] = None
        self._free.append(page)          # back of the list; it comes round again

    def owner(self, page: int):
        return self._owner[page]

    def snapshot(self) -> dict:
        return {"total": self.total, "free": self.free, "used": self.used, "peak": self.peak_used,
                "allocations": self.allocations, "failed": self.failed_allocations}


@dataclass
class RequestCache:
    slot: int
    length: int = 0                                   # tokens whose keys are in the cache
    tables: List[List[int]] = field(default_factory=list)   # per group: block -> page or FREED
    version: int = 0                                  # bumped whenever a table changes


class CacheManager:
    """Pages and slots of the live requests.

    ``groups``: the distinct paged needs (one :class:`CacheSpec` each); ``pages_per_group``:
    pool sizes. ``open`` gives a request a state slot, ``reserve`` the pages its next
    tokens need (all groups or nothing), ``commit`` advances its length and returns pages
    the window has passed, ``close`` returns everything.
    """

    def __init__(self, groups: Sequence[CacheSpec], pages_per_group: Sequence[int], page_size: int,
                 max_requests: int):
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        if len(groups) != len(pages_per_group):
            raise ValueError("one pool size per group is needed")
        self.groups = list(groups)
        self.page_size = page_size
        self.pools = [PagePool(n) for n in pages_per_group]
        self.max_requests = max_requests
        self._free_slots = deque(range(max_requests))
        self.requests: Dict[Hashable, RequestCache] = {}

    # ---- requests
    def open(self, request_id: Hashable) -> int:
        if request_id in self.requests:
            raise KeyError(f"request {request_id!r} is already open")
        if not self._free_slots:
            raise OutOfSlots(f"all {self.max_requests} request slots are taken")
        slot = self._free_slots.popleft()
        self.requests[request_id] = RequestCache(slot=slot, tables=[[] for _ in self.groups])
        return slot

    def close(self, request_id: Hashable) -> None:
        rc = self.requests.pop(request_id)
        for g, table in enumerate(rc.tables):
            for page in table:
                if page != FREED:
                    self.pools[g].give(page, request_id)
        self._free_slots.append(rc.slot)

    def is_open(self, request_id: Hashable) -> bool:
        return request_id in self.requests

    def length(self, request_id: Hashable) -> int:
        return self.requests[request_id].length

    def slot(self, request_id: Hashable) -> int:
        return self.requests[request_id].slot

    @property
    def free_slots(self) -> int:
        return len(self._free_slots)

    # ---- pages
    def _blocks_for(self, length: int, n_new: int) -> int:
        """Blocks a table must hold to cover positions < length + n_new."""
        return (length + n_new + self.page_size - 1) // self.page_size

    def pages_needed(self, request_id: Optional[Hashable], n_new: int, length: Optional[int] = None) -> List[int]:
        """New pages per group for the next ``n_new`` tokens (of an open request, or of a
        request that would start at ``length``)."""
        if request_id is not None and request_id in self.requests:
            rc = self.requests[request_id]
            have = [len(t) for t in rc.tables]
            length = rc.length
        else:
            have = [0] * len(self.groups)
            length = length or 0
        need_blocks = self._blocks_for(length, n_new)
        out = []
        for g, spec in enumerate(self.groups):
            first_live = spec.first_live_position(length) // self.page_size
            out.append(max(0, need_blocks - max(have[g], first_live)))
        return out

    def can_reserve(self, request_id: Optional[Hashable], n_new: int, length: Optional[int] = None,
                    held_back: Optional[Sequence[int]] = None) -> bool:
        need = self.pages_needed(request_id, n_new, length)
        return all(n <= self.pools[g].free - (held_back[g] if held_back else 0) for g, n in enumerate(need))

    def reserve(self, request_id: Hashable, n_new: int) -> None:
        """Pages for positions ``length .. length + n_new - 1`` in every group, or none at all."""
        rc = self.requests[request_id]
        need = self.pages_needed(request_id, n_new)
        for g, n in enumerate(need):
            if n > self.pools[g].free:
                self.pools[g].failed_allocations += 1
                raise OutOfPages(g, n, self.pools[g].free, self.pools[g].total)
        need_blocks = self._blocks_for(rc.length, n_new)
        for g, spec in enumerate(self.groups):
            table = rc.tables[g]
            first_live = spec.first_live_position(rc.length) // self.page_size
            if len(table) < need_blocks:
                rc.version += 1
            while len(table) < need_blocks:
                # blocks wholly before the window of the first new token are never read
                table.append(FREED if len(table) < first_live else self.pools[g].take(request_id))

    def commit(self, request_id: Hashable, n_new: int) -> List[Tuple[int, int]]:
        """The step ran: the request is ``n_new`` tokens longer. Pages whose every position
        lies before the window of the next token go back; returns them as (group, page)."""
        rc = self.requests[request_id]
        rc.length += n_new
        returned = []
        for g, spec in enumerate(self.groups):
            dead_blocks = spec.first_live_position(rc.length) // self.page_size
            table = rc.tables[g]
            for b in range(min(dead_blocks, len(table))):
                if table[b] != FREED:
                    self.pools[g].give(table[b], request_id)
                    returned.append((g, table[b]))
                    table[b] = FREED
                    rc.version += 1
        return returned

    def table(self, group: int, request_id: Hashable) -> List[int]:
        return self.requests[request_id].tables[group]

    def table_version(self, request_id: Hashable) -> int:
        return self.requests[request_id].version

    def held_pages(self, request_id: Hashable) -> List[int]:
        return [sum(1 for p in t if p != FREED) for t in self.requests[request_id].tables]

    def snapshot(self) -> dict:
        return {"page_size": self.page_size, "requests": len(self.requests), "free_slots": self.free_slots,
                "groups": [dict(window=spec.window, **pool.snapshot()) for spec, pool in zip(self.groups, self.pools)]}

    def check_invariants(self) -> None:
        """No page lost, held twice or free while held (tests call this after every move)."""
        for g, pool in enumerate(self.pools):
            held = {}
            for rid, rc in self.requests.items():
                for page in rc.tables[g]:
                    if page == FREED:
                        continue
                    assert page not in held, f"group {g}: page {page} held by {held[page]!r} and {rid!r}"
                    held[page] = rid
                    assert pool.owner(page) == rid, f"group {g}: page {page} owner mismatch"
            free = list(pool._free)
            assert len(set(free)) == len(free), f"group {g}: a page is on the free list twice"
            assert not (set(free) & set(held)), f"group {g}: a held page is on the free list"
            assert len(free) + len(held) == pool.total, f"group {g}: {pool.total - len(free) - len(held)} page(s) lost"
        slots = [rc.slot for rc in self.requests.values()]
        assert len(set(slots)) == len(slots), "a state slot is held twice"
        assert len(set(self._free_slots) | set(slots)) == self.max_requests, "a state slot is lost"

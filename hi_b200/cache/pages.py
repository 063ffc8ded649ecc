"""Host side of the cache: pages, block tables, state slots. The work is done by the native
host runtime (``hi_b200/csrc/host/cache.cpp``, loaded through :mod:`hi_b200.host.build`);
this module is its Python face: request ids of any hashable kind, exceptions, views.

Layer groups with different needs (every earlier key, or a window of them) have pools of
their own; a request has one block table per group, indexed by ``position // page_size``.
Pages go back to their pool when the request ends or when the window has passed them, and
are handed out again (the reference allocates everything at admission and frees only at
retirement: crates/hi-cuda/src/lib.rs:641-957, 4781-4844).
"""
from __future__ import annotations

import ctypes
from typing import Dict, Hashable, Iterator, List, Optional, Sequence, Tuple

import numpy as np

from ..host import build as host
from ..parts.spec import CacheSpec

FREED = -1   # a block whose page was given back (the window has passed it)
_WINDOW_KINDS = {"chunk": 1, "sliding": 2}


class OutOfPages(RuntimeError):
    """insufficient_gpu_memory in the reference's terms (crates/hi-cuda/src/lib.rs:845-858)."""

    def __init__(self, group: int, needed: int, free: int, total: int):
        super().__init__(f"insufficient_gpu_memory: page group {group} needs {needed} page(s), "
                         f"only {free} of {total} free")
        self.group, self.needed, self.free, self.total = group, needed, free, total


class OutOfSlots(RuntimeError):
    pass


class _Handles:
    """Request ids (any hashable) <-> the 64-bit handles the native runtime works with. A handle
    is never used twice; an id keeps its handle while the request is open in the cache or pinned
    (known to a scheduler)."""

    def __init__(self):
        self.of_id: Dict[Hashable, int] = {}
        self.of_handle: Dict[int, Hashable] = {}
        self.pinned: Dict[int, int] = {}
        self._next = 0

    def get(self, rid: Hashable) -> Optional[int]:
        return self.of_id.get(rid)

    def make(self, rid: Hashable) -> int:
        h = self.of_id.get(rid)
        if h is None:
            h = self._next
            self._next += 1
            self.of_id[rid] = h
            self.of_handle[h] = rid
        return h

    def pin(self, rid: Hashable) -> int:
        h = self.make(rid)
        self.pinned[h] = self.pinned.get(h, 0) + 1
        return h

    def unpin(self, h: int) -> None:
        n = self.pinned.get(h, 0) - 1
        if n > 0:
            self.pinned[h] = n
        else:
            self.pinned.pop(h, None)

    def drop_if_unused(self, h: int, still_open: bool) -> None:
        if not still_open and h not in self.pinned:
            rid = self.of_handle.pop(h, None)
            if rid is not None:
                self.of_id.pop(rid, None)


class PagePool:
    """Free list of one group. Every page has at most one owner; giving back a page that is
    not held, or not held by that owner, raises."""

    def __init__(self, num_pages: int, _borrowed=None, _handles: Optional[_Handles] = None):
        self._lib = host.library()
        if _borrowed is None:
            if num_pages <= 0:
                raise ValueError("a page pool needs at least one page")
            self._ptr = self._lib.hbh_pool_create(int(num_pages))
            self._owned = True
        else:
            self._ptr, self._owned = _borrowed, False
        self._handles = _handles if _handles is not None else _Handles()

    def __del__(self):
        if getattr(self, "_owned", False) and self._ptr:
            self._lib.hbh_pool_destroy(self._ptr)
            self._ptr = None

    def _stat(self, what: int) -> int:
        return int(self._lib.hbh_pool_stat(self._ptr, what))

    total = property(lambda self: self._stat(0))
    free = property(lambda self: self._stat(1))
    used = property(lambda self: self._stat(2))
    peak_used = property(lambda self: self._stat(3))
    allocations = property(lambda self: self._stat(4))
    failed_allocations = property(lambda self: self._stat(5))

    def take(self, owner: Hashable) -> int:
        page = ctypes.c_int(-1)
        code = self._lib.hbh_pool_take(self._ptr, self._handles.make(owner), ctypes.byref(page))
        if code == host.ERR_NO_PAGES:
            raise OutOfPages(-1, 1, 0, self.total)
        return page.value

    def give(self, page: int, owner: Hashable) -> None:
        h = self._handles.get(owner)
        code = self._lib.hbh_pool_give(self._ptr, int(page), -1 if h is None else h)
        if code == host.ERR_BAD_PAGE:
            raise ValueError(f"page {page} is outside the pool")
        if code == host.ERR_DOUBLE_FREE:
            raise RuntimeError(f"page {page} freed twice")
        if code == host.ERR_NOT_OWNER:
            raise RuntimeError(f"page {page} is held by {self.owner(page)!r}, not by {owner!r}")

    def owner(self, page: int):
        h, held = ctypes.c_int64(0), ctypes.c_int(0)
        if self._lib.hbh_pool_owner(self._ptr, int(page), ctypes.byref(h), ctypes.byref(held)) != host.OK:
            raise ValueError(f"page {page} is outside the pool")
        return self._handles.of_handle.get(h.value) if held.value else None

    def snapshot(self) -> dict:
        return {"total": self.total, "free": self.free, "used": self.used, "peak": self.peak_used,
                "allocations": self.allocations, "failed": self.failed_allocations}


class RequestCache:
    """A read-only picture of one open request: slot, length, block tables (copies), table version."""

    __slots__ = ("slot", "length", "tables", "version")

    def __init__(self, slot: int, length: int, tables: List[List[int]], version: int):
        self.slot, self.length, self.tables, self.version = slot, length, tables, version


class _OpenRequests:
    """``manager.requests``: the open requests as a read-only mapping id -> :class:`RequestCache`."""

    def __init__(self, manager: "CacheManager"):
        self._m = manager

    def _ids(self) -> List[Hashable]:
        m = self._m
        n = m._lib.hbh_cache_open_requests(m._ptr, None, 0)
        buf = (ctypes.c_int64 * max(n, 1))()
        m._lib.hbh_cache_open_requests(m._ptr, buf, n)
        return [m._handles.of_handle[buf[i]] for i in range(n)]

    def __len__(self) -> int:
        return self._m._lib.hbh_cache_open_requests(self._m._ptr, None, 0)

    def __bool__(self) -> bool:
        return len(self) > 0

    def __contains__(self, rid: Hashable) -> bool:
        return self._m.is_open(rid)

    def __iter__(self) -> Iterator[Hashable]:
        return iter(self._ids())

    def keys(self):
        return self._ids()

    def __getitem__(self, rid: Hashable) -> RequestCache:
        m = self._m
        h = m._open_handle(rid)
        return RequestCache(m.slot(rid), m.length(rid), [m.table(g, rid) for g in range(len(m.groups))],
                            int(m._lib.hbh_cache_request_stat(m._ptr, h, 2)))

    def items(self):
        return [(rid, self[rid]) for rid in self._ids()]

    def values(self):
        return [self[rid] for rid in self._ids()]


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
        if any(int(n) <= 0 for n in pages_per_group):
            raise ValueError("a page pool needs at least one page")
        self.groups = list(groups)
        self.page_size = int(page_size)
        self.max_requests = int(max_requests)
        kinds, sizes = [], []
        for spec in self.groups:
            if spec.window is None:
                kinds.append(0); sizes.append(0)
            else:
                kind, size = spec.window
                if kind not in _WINDOW_KINDS or int(size) <= 0:
                    raise ValueError(f"unknown cache window {spec.window!r}")
                kinds.append(_WINDOW_KINDS[kind]); sizes.append(int(size))
        n = len(self.groups)
        self._lib = host.library()
        self._ptr = self._lib.hbh_cache_create(
            n, (ctypes.c_int * max(n, 1))(*kinds), (ctypes.c_int64 * max(n, 1))(*sizes),
            (ctypes.c_int * max(n, 1))(*[int(p) for p in pages_per_group]), self.page_size, self.max_requests)
        if not self._ptr:
            raise ValueError("the native cache manager refused these sizes")
        self._handles = _Handles()
        self.pools = [PagePool(0, _borrowed=self._lib.hbh_cache_pool(self._ptr, g), _handles=self._handles)
                      for g in range(n)]
        self.requests = _OpenRequests(self)
        self._need = (ctypes.c_int * max(n, 1))()
        self._fail = (ctypes.c_int * 4)()

    def __del__(self):
        if getattr(self, "_ptr", None):
            self._lib.hbh_cache_destroy(self._ptr)
            self._ptr = None

    # ---- handles
    def _open_handle(self, rid: Hashable) -> int:
        h = self._handles.get(rid)
        if h is None or not self._lib.hbh_cache_is_open(self._ptr, h):
            raise KeyError(rid)
        return h

    # ---- requests
    def open(self, request_id: Hashable) -> int:
        h = self._handles.make(request_id)
        slot = ctypes.c_int(-1)
        code = self._lib.hbh_cache_open(self._ptr, h, ctypes.byref(slot))
        if code == host.ERR_ALREADY_OPEN:
            raise KeyError(f"request {request_id!r} is already open")
        if code == host.ERR_NO_SLOT:
            self._handles.drop_if_unused(h, False)
            raise OutOfSlots(f"all {self.max_requests} request slots are taken")
        return slot.value

    def close(self, request_id: Hashable) -> None:
        h = self._open_handle(request_id)
        code = self._lib.hbh_cache_close(self._ptr, h)
        self._handles.drop_if_unused(h, False)
        if code != host.OK:
            raise RuntimeError(f"closing {request_id!r}: a page could not be given back (code {code})")

    def is_open(self, request_id: Hashable) -> bool:
        h = self._handles.get(request_id)
        return h is not None and bool(self._lib.hbh_cache_is_open(self._ptr, h))

    def length(self, request_id: Hashable) -> int:
        return int(self._lib.hbh_cache_request_stat(self._ptr, self._open_handle(request_id), 1))

    def slot(self, request_id: Hashable) -> int:
        return int(self._lib.hbh_cache_request_stat(self._ptr, self._open_handle(request_id), 0))

    @property
    def free_slots(self) -> int:
        return self._lib.hbh_cache_free_slots(self._ptr)

    # ---- pages
    def pages_needed(self, request_id: Optional[Hashable], n_new: int, length: Optional[int] = None) -> List[int]:
        """New pages per group for the next ``n_new`` tokens (of an open request, or of a
        request that would start at ``length``)."""
        h = self._handles.get(request_id) if request_id is not None else None
        self._lib.hbh_cache_pages_needed(self._ptr, -1 if h is None else h, int(n_new), int(length or 0), self._need)
        return list(self._need[: len(self.groups)])

    def can_reserve(self, request_id: Optional[Hashable], n_new: int, length: Optional[int] = None,
                    held_back: Optional[Sequence[int]] = None) -> bool:
        need = self.pages_needed(request_id, n_new, length)
        return all(n <= self.pools[g].free - (held_back[g] if held_back else 0) for g, n in enumerate(need))

    def reserve(self, request_id: Hashable, n_new: int) -> None:
        """Pages for positions ``length .. length + n_new - 1`` in every group, or none at all."""
        code = self._lib.hbh_cache_reserve(self._ptr, self._open_handle(request_id), int(n_new), self._fail)
        if code == host.ERR_NO_PAGES:
            raise OutOfPages(*self._fail[:4])
        if code != host.OK:
            raise RuntimeError(f"reserve failed with code {code}")

    def table_lengths(self, request_id: Hashable) -> List[int]:
        h = self._open_handle(request_id)
        return [self._lib.hbh_cache_table_length(self._ptr, g, h) for g in range(len(self.groups))]

    def unreserve(self, request_id: Hashable, table_lengths: Sequence[int]) -> None:
        """Undo a reserve: the tables shrink back to ``table_lengths``, the pages beyond return."""
        n = len(self.groups)
        code = self._lib.hbh_cache_unreserve(self._ptr, self._open_handle(request_id),
                                             (ctypes.c_int * max(n, 1))(*[int(x) for x in table_lengths]))
        if code != host.OK:
            raise RuntimeError(f"unreserve failed with code {code}")

    def commit(self, request_id: Hashable, n_new: int) -> List[Tuple[int, int]]:
        """The step ran: the request is ``n_new`` tokens longer. Pages whose every position
        lies before the window of the next token go back; returns them as (group, page)."""
        n = self._lib.hbh_cache_commit(self._ptr, self._open_handle(request_id), int(n_new))
        if n < 0:
            raise RuntimeError(f"commit failed with code {n}")
        if n == 0:
            return []
        buf = (ctypes.c_int * (2 * n))()
        self._lib.hbh_cache_returned(self._ptr, buf, n)
        return [(buf[2 * i], buf[2 * i + 1]) for i in range(n)]

    def table(self, group: int, request_id: Hashable) -> List[int]:
        h = self._open_handle(request_id)
        n = self._lib.hbh_cache_table_length(self._ptr, group, h)
        if n < 0:
            raise IndexError(group)
        buf = (ctypes.c_int * max(n, 1))()
        self._lib.hbh_cache_table(self._ptr, group, h, buf, n)
        return list(buf[:n])

    def table_version(self, request_id: Hashable) -> int:
        return int(self._lib.hbh_cache_request_stat(self._ptr, self._open_handle(request_id), 2))

    def held_pages(self, request_id: Hashable) -> List[int]:
        return [sum(1 for p in self.table(g, request_id) if p != FREED) for g in range(len(self.groups))]

    def snapshot(self) -> dict:
        return {"page_size": self.page_size, "requests": len(self.requests), "free_slots": self.free_slots,
                "groups": [dict(window=spec.window, **pool.snapshot()) for spec, pool in zip(self.groups, self.pools)]}

    def check_invariants(self) -> None:
        """No page lost, held twice or free while held (tests call this after every move)."""
        if self._lib.hbh_cache_check(self._ptr) != host.OK:
            raise AssertionError(self._lib.hbh_cache_error(self._ptr).decode())

    # ---- a step's integer inputs
    def step_widths(self, handles: np.ndarray) -> List[int]:
        n = len(self.groups)
        out = (ctypes.c_int * max(n, 1))()
        code = self._lib.hbh_step_widths(self._ptr, len(handles), handles.ctypes.data, out)
        if code != host.OK:
            raise KeyError("a request of the step is not open")
        return list(out[:n])

    def handles_of(self, request_ids: Sequence[Hashable]) -> np.ndarray:
        return np.array([self._open_handle(r) for r in request_ids], dtype=np.int64)

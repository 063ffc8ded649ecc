"""Device side of the cache: per cache slot a key pool and a value pool of pages, per
mixer with fixed-size state a [max_requests, ...] tensor.

Page layout [pages, kv_heads, page_size, head_dim] (one kv head's page_size rows are
contiguous; address rule as crates/hi-cuda/src/kernels.cu:4214-4219). One page id addresses
the same place in every cache slot of its group.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..parts.context import CacheView
from ..parts.spec import CacheSpec


def plan_groups(cache_specs: Dict[int, Optional[CacheSpec]]) -> Tuple[List[CacheSpec], Dict[int, int]]:
    """Distinct paged needs -> groups; returns (one spec per group, group of each cache slot)."""
    groups: List[CacheSpec] = []
    keys: Dict[tuple, int] = {}
    group_of: Dict[int, int] = {}
    for slot in sorted(cache_specs):
        spec = cache_specs[slot]
        if spec is None or not spec.paged:
            continue
        if spec.group_key not in keys:
            keys[spec.group_key] = len(groups)
            groups.append(CacheSpec(kv_heads=spec.kv_heads, head_dim=spec.head_dim, window=spec.window))
        group_of[slot] = keys[spec.group_key]
    return groups, group_of


def bytes_per_token(cache_specs: Dict[int, Optional[CacheSpec]], element_size: int) -> List[int]:
    """Per group: bytes one cached token takes in all the cache slots of the group (keys and values)."""
    groups, group_of = plan_groups(cache_specs)
    out = [0] * len(groups)
    for slot, spec in cache_specs.items():
        if spec is not None and spec.paged:
            out[group_of[slot]] += 2 * spec.kv_heads * spec.head_dim * element_size
    return out


def pool_tokens_for_budget(cache_specs: Dict[int, Optional[CacheSpec]], element_size: int, budget_bytes: int,
                           page_size: int, max_requests: int, most_tokens: Optional[int] = None,
                           portion_tokens: int = 8192) -> List[int]:
    """Pool sizes (tokens per group) from a byte budget (the reference sizes its one pool from the
    token budget of a step, crates/hi-cuda/src/lib.rs:794-797; here the memory that is free decides).
    A windowed group never holds more than its window, the page being written and the portion in
    flight for every request, so it gets that (or less, if the budget is smaller); what is left
    goes to the groups that keep every key, in proportion to what a token costs them. ``most_tokens``
    caps the result (``max_requests`` requests at the model's longest context need no more)."""
    groups, _ = plan_groups(cache_specs)
    cost = bytes_per_token(cache_specs, element_size)
    if not groups:
        return []
    floor = page_size * max(2, max_requests)                     # never less than two pages a request could take
    tokens = [0] * len(groups)
    left = int(budget_bytes)
    windowed = [g for g, spec in enumerate(groups) if spec.window is not None]
    keep_all = [g for g, spec in enumerate(groups) if spec.window is None]
    for g in windowed:
        want = max_requests * (groups[g].window[1] + 2 * page_size) + portion_tokens
        if most_tokens is not None:
            want = min(want, most_tokens)
        share = left // max(1, len(windowed) + len(keep_all)) if keep_all else left // len(windowed)
        tokens[g] = max(floor, min(want, share // cost[g]))
        left -= tokens[g] * cost[g]
    if keep_all:
        per_token = sum(cost[g] for g in keep_all)
        t = max(floor, left // per_token)
        if most_tokens is not None:
            t = min(t, max(most_tokens, floor))
        for g in keep_all:
            tokens[g] = t
    return [-(-t // page_size) * page_size for t in tokens]


class DeviceCache:
    def __init__(self, cache_specs: Dict[int, Optional[CacheSpec]], pages_per_group: Sequence[int], page_size: int,
                 max_requests: int, dtype: torch.dtype, device):
        self.groups, self.group_of = plan_groups(cache_specs)
        self.page_size, self.dtype, self.device = page_size, dtype, torch.device(device)
        self.views: Dict[int, CacheView] = {}
        self.bytes = 0
        for slot, spec in cache_specs.items():
            view = CacheView()
            if spec is not None and spec.paged:
                g = self.group_of[slot]
                shape = (pages_per_group[g], spec.kv_heads, page_size, spec.head_dim)
                view.group = g
                view.k_pages = torch.zeros(shape, dtype=dtype, device=self.device)
                view.v_pages = torch.zeros(shape, dtype=dtype, device=self.device)
                self.bytes += 2 * view.k_pages.numel() * view.k_pages.element_size()
            if spec is not None and spec.state_shape:
                sdt = getattr(torch, spec.state_dtype)
                view.state = torch.zeros((max_requests, *spec.state_shape), dtype=sdt, device=self.device)
                self.bytes += view.state.numel() * view.state.element_size()
            self.views[slot] = view

    def reset_slot(self, slot: int) -> None:
        """A request's fixed-size state starts at zero."""
        for view in self.views.values():
            if view.state is not None:
                view.state[slot].zero_()

    def poison_pages(self, returned) -> None:
        """Debug aid: fill returned pages with NaN so a read of a freed page shows."""
        by_group: Dict[int, List[int]] = {}
        for g, page in returned:
            by_group.setdefault(g, []).append(page)
        for slot, view in self.views.items():
            pages = by_group.get(view.group) if view.group is not None else None
            if pages:
                idx = torch.tensor(pages, device=self.device, dtype=torch.long)
                view.k_pages[idx] = float("nan")
                view.v_pages[idx] = float("nan")

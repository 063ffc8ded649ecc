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

"""What the step function hands to the parts: the batch of one step, and a mixer's cache."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

import torch


@dataclass
class StepContext:
    """One step: N new tokens of S requests, flat. All tensors live on the device.

    Request ``s`` contributes ``n_new[s]`` consecutive tokens at positions
    ``start_pos[s] ..``; rows ``cu_seqlens[s] .. cu_seqlens[s+1]`` of every [N, ...] tensor
    are its tokens. ``slots[s]`` is the request's fixed-size state slot.
    """

    n_tokens: int
    n_seqs: int
    tokens: torch.Tensor          # int32 [N]
    positions: torch.Tensor       # int32 [N]  absolute position of each token
    seq_of_token: torch.Tensor    # int32 [N]  row of the block tables / index into slots
    cu_seqlens: torch.Tensor      # int32 [S+1]
    slots: torch.Tensor           # int32 [S]
    start_pos: List[int]          # host copies
    n_new: List[int]
    slot_ids: List[int]
    block_tables: Dict[int, torch.Tensor] = field(default_factory=dict)   # group -> int32 [S, width]
    page_size: int = 0
    max_context: int = 0          # longest start_pos + n_new in the step
    tap: Optional[Callable[[str, torch.Tensor], None]] = None   # debug: parts report named tensors
    # debug: choices a part is told to take instead of its own, by the name it reports them under
    # (the router's expert ids, int32 [N, k] in the step's flat token order)
    forced: Optional[Dict[str, torch.Tensor]] = None
    # mixed steps only: flat rows of the requests that bring ONE token (int64 [D]) and the longest
    # context among them; None when the step is all portions or all single tokens
    decode_rows: Optional[torch.Tensor] = None
    decode_max_context: int = 0

    @property
    def max_new(self) -> int:
        return max(self.n_new) if self.n_new else 0


@dataclass
class CacheView:
    """The cache slot of one schedule entry, as its mixer sees it."""

    group: Optional[int] = None                  # page group (None: no paged cache)
    k_pages: Optional[torch.Tensor] = None       # [pages, kv_heads, page_size, head_dim]
    v_pages: Optional[torch.Tensor] = None
    state: Optional[torch.Tensor] = None         # [max_slots, *state_shape]
    writes: bool = True                          # False: read another entry's cache, do not append


@dataclass
class Pending:
    """A sub-layer's output that has not yet been added to the residual stream: a dense part
    (engine dtype or float32, [N, H]) and/or the routed experts' rows (float32 [N*k, H] in
    expert-sorted order, with the slot of every (token, rank) entry). The next norm adds all of
    it in one pass."""

    dense: Optional[torch.Tensor] = None
    routed: Optional[torch.Tensor] = None
    slot_of_entry: Optional[torch.Tensor] = None
    top_k: int = 0
    entry_weights: Optional[torch.Tensor] = None     # float32 [N*k]: factors of the routed rows in the sum

    def materialize(self, n_tokens: int) -> torch.Tensor:
        """The sum as one float32 tensor, for a consumer that is not a norm."""
        from ..kernels import ops

        if self.routed is None:
            return self.dense
        return ops.moe_combine(self.routed, self.slot_of_entry, self.dense, n_tokens, self.top_k, self.entry_weights)

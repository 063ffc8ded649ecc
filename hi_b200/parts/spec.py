"""A model as data: parts chosen layer by layer, and the order in which layers run.

Nothing here knows an architecture. An architecture's builder (for instance
``hi_b200/config/registry.py`` -> ``hi_b200/parts/llama4.py``) turns its typed
configuration into a :class:`ModelSpec`; ``hi_b200/parts/model.py`` instantiates it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part: the name it is registered under and its sizes and constants."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class TensorSpec:
    """A tensor a part wants from the checkpoint.

    ``init`` drives the random-weights writer: "normal" (N(0, std)), "ones", "zeros".
    ``dtype`` is "float" (stored bf16, kept bf16 or widened in the 32-bit path) or
    "int32" (integer tables).
    """

    name: str
    shape: Tuple[int, ...]
    init: str = "normal"
    dtype: str = "float"
    optional: bool = False


@dataclass(frozen=True)
class CacheSpec:
    """What a mixer keeps between steps.

    Per token: one key row and one value row of ``kv_heads * head_dim`` elements,
    kept for ``window``: ``None`` = all earlier tokens, ``("chunk", C)`` = tokens of
    the query's own block of C positions, ``("sliding", W)`` = the last W tokens.
    Per request: ``state_shape`` elements of fixed size (``()`` = none).
    Mixers with equal paged needs share a page group (one block table per request).
    """

    kv_heads: int = 0
    head_dim: int = 0
    window: Optional[Tuple[str, int]] = None
    state_shape: Tuple[int, ...] = ()
    state_dtype: str = "float32"

    @property
    def paged(self) -> bool:
        return self.kv_heads > 0 and self.head_dim > 0

    @property
    def group_key(self):
        return (self.kv_heads, self.head_dim, self.window)

    def first_live_position(self, next_position: int) -> int:
        """Oldest position a query at ``next_position`` or later can still read."""
        if self.window is None:
            return 0
        kind, size = self.window
        if kind == "chunk":
            return (next_position // size) * size
        if kind == "sliding":
            return max(0, next_position - size + 1)
        raise ValueError(f"unknown cache window kind {kind!r}")


@dataclass(frozen=True)
class LayerSpec:
    """One layer: its parts and how the block arranges them."""

    prefix: str                      # tensor-name prefix, e.g. "model.layers.3"
    mixer: PartSpec
    feed_forward: PartSpec
    norm_mixer: PartSpec
    norm_feed_forward: PartSpec
    arrangement: str = "prenorm"


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer. ``cache`` names the cache slot its mixer uses; two entries
    with the same ``cache`` share it, and only entries with ``writes_cache`` append."""

    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    eos_token_ids: Tuple[int, ...] = ()
    max_position_embeddings: Optional[int] = None

    @staticmethod
    def sequential(n_layers: int) -> Tuple[ScheduleEntry, ...]:
        return tuple(ScheduleEntry(layer=i, cache=i) for i in range(n_layers))

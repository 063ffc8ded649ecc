"""Registries of parts by name. A part registers itself with ``@register(family, name)``;
a model is assembled from :class:`~hi_b200.parts.spec.PartSpec` entries by :func:`build`.

Families and the interface each member must have (all also have
``tensor_specs() -> list[TensorSpec]`` and ``load(tensors: dict[str, Tensor])``):

``norm``          ``forward(residual_f32, delta_or_None) -> normed``: adds ``delta`` into
                  the 32-bit residual stream in place first, then normalises.
``position``      ``rotary_table() -> (inv_freq_f32 [rot/2], interleaved) | None`` for the
                  fused kernel, or ``apply(q, k, positions) -> (q, k)`` for anything else.
``mixer``         ``cache_spec() -> CacheSpec | None``;
                  ``forward(normed, ctx, cache_view) -> delta``.
``feed_forward``  ``forward(normed, ctx) -> delta`` (engine dtype or float32).
``arrangement``   ``forward(layer, residual, pending, ctx, cache_view) -> (residual, pending)``.
``embedding``     ``forward(tokens_i32) -> residual_f32``; ``table`` for a tied head.
``head``          ``forward(normed_rows) -> logits_f32``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict

import torch

from .spec import PartSpec

FAMILIES = ("norm", "position", "mixer", "feed_forward", "arrangement", "embedding", "head")
_REGISTRY: Dict[str, Dict[str, Callable[..., Any]]] = {f: {} for f in FAMILIES}


@dataclass(frozen=True)
class BuildEnv:
    """What every part is told when it is built."""

    dtype: torch.dtype          # torch.bfloat16 (serving) or torch.float32 (true 32-bit path)
    device: torch.device
    hidden_size: int


def register(family: str, name: str):
    if family not in _REGISTRY:
        raise KeyError(f"unknown part family {family!r}; families: {FAMILIES}")

    def deco(cls):
        _REGISTRY[family][name] = cls
        return cls

    return deco


def unregister(family: str, name: str) -> None:
    _REGISTRY[family].pop(name, None)


def registered(family: str):
    return sorted(_REGISTRY[family])


def build(family: str, spec: PartSpec, env: BuildEnv, prefix: str = ""):
    try:
        cls = _REGISTRY[family][spec.kind]
    except KeyError:
        raise KeyError(
            f"no {family} part named {spec.kind!r} is registered; known: {registered(family)}") from None
    return cls(dict(spec.params), prefix, env)

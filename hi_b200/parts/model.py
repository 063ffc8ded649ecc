"""A decoder assembled from a :class:`ModelSpec`: embedding, a schedule of layers, final norm, head."""
from __future__ import annotations

from typing import Callable, Dict, List, Optional

import torch

from . import attention as _attention  # noqa: F401  (registers the parts)
from . import basic as _basic          # noqa: F401
from . import feed_forward as _ffn     # noqa: F401
from .context import CacheView, StepContext
from .registry import BuildEnv, build
from .spec import CacheSpec, ModelSpec, PartSpec, TensorSpec


class Layer:
    """The parts of one layer, built from its :class:`LayerSpec`."""

    def __init__(self, spec, env: BuildEnv):
        self.spec = spec

        def sub(part_spec):
            name = part_spec.params.get("name")
            return f"{spec.prefix}.{name}" if name else spec.prefix

        self.norm_mixer = build("norm", spec.norm_mixer, env, sub(spec.norm_mixer))
        self.mixer = build("mixer", spec.mixer, env, sub(spec.mixer))
        self.norm_feed_forward = build("norm", spec.norm_feed_forward, env, sub(spec.norm_feed_forward))
        self.feed_forward = build("feed_forward", spec.feed_forward, env, sub(spec.feed_forward))
        self.arrangement = build("arrangement", PartSpec(spec.arrangement), env, spec.prefix)

    def parts(self):
        return [self.norm_mixer, self.mixer, self.norm_feed_forward, self.feed_forward]


class Model:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype {dtype} is not supported (bfloat16 or float32)")
        self.spec, self.dtype, self.device = spec, dtype, torch.device(device)
        self.env = BuildEnv(dtype=dtype, device=self.device, hidden_size=spec.hidden_size)
        self.embedding = build("embedding", spec.embedding, self.env, spec.embedding.params.get("name", ""))
        self.layers = [Layer(ls, self.env) for ls in spec.layers]
        self.final_norm = build("norm", spec.final_norm, self.env, spec.final_norm.params.get("name", ""))
        self.head = build("head", spec.head, self.env, spec.head.params.get("name", ""))
        for i, entry in enumerate(spec.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"schedule entry {i} names layer {entry.layer}; the model has {len(self.layers)}")
        # cache slots: the spec of the mixer of the first entry that names the slot
        self.cache_specs: Dict[int, Optional[CacheSpec]] = {}
        for entry in spec.schedule:
            cs = self.layers[entry.layer].mixer.cache_spec()
            if entry.cache in self.cache_specs:
                if self.cache_specs[entry.cache] != cs:
                    raise ValueError(f"cache slot {entry.cache} is shared by mixers with different cache needs")
            else:
                self.cache_specs[entry.cache] = cs
        writers = {e.cache for e in spec.schedule if e.writes_cache}
        for slot in self.cache_specs:
            if slot not in writers:
                raise ValueError(f"cache slot {slot} is read but no schedule entry writes it")
        self.loaded = False
        self.graph_safe = all(getattr(p, "graph_safe", False) for p in self.all_parts()) and \
            all(getattr(l.arrangement, "graph_safe", False) for l in self.layers)

    # ---- weights
    def all_parts(self):
        parts = [self.embedding]
        for layer in self.layers:
            parts += layer.parts()
        return parts + [self.final_norm, self.head]

    def tensor_specs(self) -> List[TensorSpec]:
        specs: List[TensorSpec] = []
        for part in self.all_parts():
            specs += part.tensor_specs()
        return specs

    def load(self, fetch: Callable[[str], Optional[torch.Tensor]]) -> None:
        for part in self.all_parts():
            part.load(fetch)
        self.loaded = True

    # ---- one step
    def forward(self, ctx: StepContext, caches: Dict[int, CacheView], logit_rows: Optional[torch.Tensor]):
        """Run the step's tokens through the schedule; float32 logits [len(logit_rows), V]
        (None when no logits are wanted: the final norm and the head are then skipped)."""
        if not self.loaded:
            raise RuntimeError("model weights are not loaded")
        residual = self.embedding.forward(ctx.tokens)
        pending = None
        for entry in self.spec.schedule:
            layer = self.layers[entry.layer]
            view = caches[entry.cache]
            if view.writes != entry.writes_cache:
                view = CacheView(group=view.group, k_pages=view.k_pages, v_pages=view.v_pages, state=view.state,
                                 writes=entry.writes_cache)
            residual, pending = layer.arrangement.forward(layer, residual, pending, ctx, view)
        if logit_rows is None or logit_rows.numel() == 0:
            return None
        z = self.final_norm.forward(residual, pending, logit_rows)
        return self.head.forward(z, self.embedding)

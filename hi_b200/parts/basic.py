"""Norm, position encoding, embedding, output head and the block arrangement."""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import numpy as np
import torch

from ..kernels import ops
from .context import Pending
from .linear import linear
from .registry import BuildEnv, build, register
from .spec import PartSpec, TensorSpec


class Part:
    """Common shape of a part: parameters in, tensors by name, nothing model-specific.

    ``graph_safe``: the part's forward only enqueues work whose shape depends on the number of
    tokens and reads the step's device tensors, never its host-side lists; a decode step made of
    such parts may be captured in a CUDA graph. A part that does not say so is never captured."""

    graph_safe = False

    def __init__(self, params: dict, prefix: str, env: BuildEnv):
        self.params, self.prefix, self.env = params, prefix, env

    def tensor_specs(self) -> List[TensorSpec]:
        return []

    def load(self, fetch) -> None:
        """``fetch(name)`` returns the named tensor on the device (or None if optional and absent)."""

    def cache_spec(self):
        return None


# --------------------------------------------------------------------------- norms
@register("norm", "rmsnorm")
class RMSNorm(Part):
    """y = x * rsqrt(mean(x^2) + eps) * w, statistics in float32
    (crates/hi-mlx/src/models.rs:1977-1979; crates/hi-cuda/src/kernels.cu:61-77).
    params: ``size``, ``eps``, ``name`` (tensor ``<prefix>.weight``)."""

    graph_safe = True

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.size, self.eps = int(params["size"]), float(params["eps"])
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self):
        return [TensorSpec(f"{self.prefix}.weight", (self.size,), init="ones")]

    def load(self, fetch):
        self.weight = fetch(f"{self.prefix}.weight").contiguous()

    def forward(self, residual: torch.Tensor, delta, row_map: Optional[torch.Tensor] = None, also_f32: bool = False):
        """``delta``: None, a tensor, or a :class:`~hi_b200.parts.context.Pending`."""
        if isinstance(delta, Pending):
            if delta.top_k > 8:
                delta = delta.materialize(residual.shape[0])
            else:
                return ops.add_rmsnorm(residual, delta.dense, self.weight, self.eps, self.env.dtype, row_map, also_f32,
                                       delta.routed, delta.slot_of_entry, delta.top_k, delta.entry_weights)
        return ops.add_rmsnorm(residual, delta, self.weight, self.eps, self.env.dtype, row_map, also_f32)


# --------------------------------------------------------------------------- positions
def llama3_inverse_frequencies(head_dim: int, theta: float, scaling: Optional[dict]) -> np.ndarray:
    """inv_freq[j] = theta^(-2j/hd), rescaled by parts when ``scaling`` is given
    (crates/hi-mlx/src/models.rs:5897-5926, 6166-6175), all in float32 as there. Where the
    reference would divide 0 by 0 (high == low and the wavelength exactly on the boundary)
    the low-frequency value is taken."""
    f32 = np.float32
    out = np.empty(head_dim // 2, dtype=f32)
    for j in range(head_dim // 2):
        th = np.power(f32(theta), f32((2 * j) / head_dim), dtype=f32)
        inv = f32(1.0) / th
        if scaling:
            factor, low = f32(scaling["factor"]), f32(scaling["low_freq_factor"])
            high, orig = f32(scaling["high_freq_factor"]), f32(scaling["original_max_position_embeddings"])
            wavelen = f32(2.0) * f32(math.pi) / inv
            if wavelen > orig / low:
                inv = inv / factor
            elif wavelen < orig / high:
                pass
            else:
                smooth = f32(0.0) if high == low else (orig / wavelen - low) / (high - low)
                inv = (f32(1.0) - smooth) * inv / factor + smooth * inv
        out[j] = inv
    return out


@register("position", "rope")
class RotaryPosition(Part):
    """Rotary encoding of q and k: all head_dim dims, or with ``rot_dim`` the first rot_dim of them
    (a multiple of 16; the rest pass through).
    params: ``head_dim``, ``theta``, ``scaling`` (dict or None), ``interleaved`` (pairs (2j, 2j+1)
    instead of (j, j + rot_dim/2)), ``rot_dim`` (default head_dim; the frequencies are
    theta^(-2j/rot_dim))."""

    graph_safe = True

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.interleaved = bool(params.get("interleaved", False))
        self.rot_dim = int(params.get("rot_dim") or params["head_dim"])
        if self.rot_dim % 16 or not 0 < self.rot_dim <= int(params["head_dim"]):
            raise ValueError(f"{prefix}: rot_dim {self.rot_dim} must be a multiple of 16, at most head_dim")
        self._table_host = llama3_inverse_frequencies(self.rot_dim, float(params["theta"]), params.get("scaling"))
        self._table: Optional[torch.Tensor] = None

    def rotary_table(self):
        if self._table is None:
            self._table = torch.from_numpy(self._table_host).to(self.env.device)
        return self._table, self.interleaved


@register("position", "none")
class NoPosition(Part):
    """NoPE: q and k are used as projected."""

    graph_safe = True

    def rotary_table(self):
        return None


# --------------------------------------------------------------------------- embedding and head
@register("embedding", "token_embedding")
class TokenEmbedding(Part):
    """x[t] = table[token[t]], no multiplier (crates/hi-mlx/src/models.rs:6206, 1915-1917).
    params: ``vocab_size``, ``hidden_size``; tensor ``<prefix>.weight``."""

    graph_safe = True

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.table: Optional[torch.Tensor] = None

    def tensor_specs(self):
        return [TensorSpec(f"{self.prefix}.weight", (int(self.params["vocab_size"]), int(self.params["hidden_size"])))]

    def load(self, fetch):
        self.table = fetch(f"{self.prefix}.weight").contiguous()

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        return ops.embed_gather(self.table, tokens)


@register("head", "linear_head")
class LinearHead(Part):
    """logits = z W^T in float32. The separate head is used when its tensor exists, else the
    embedding table (decided by presence, crates/hi-mlx/src/models.rs:6186-6193, 6211-6214).
    params: ``vocab_size``, ``hidden_size``, ``tie`` (random weights: write no head tensor)."""

    graph_safe = True

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.weight: Optional[torch.Tensor] = None
        self.tied = False

    def tensor_specs(self):
        # "absent": the random-weights writer leaves a tied head out of the folder
        return [TensorSpec(f"{self.prefix}.weight", (int(self.params["vocab_size"]), int(self.params["hidden_size"])),
                           init="absent" if self.params.get("tie", False) else "normal", optional=True)]

    def load(self, fetch):
        w = fetch(f"{self.prefix}.weight")
        self.tied = w is None
        self.weight = None if w is None else w.contiguous()

    def forward(self, normed_rows: torch.Tensor, embedding: TokenEmbedding) -> torch.Tensor:
        w = embedding.table if self.weight is None else self.weight
        return linear(normed_rows, w, out_dtype=torch.float32)


# --------------------------------------------------------------------------- block arrangement
@register("arrangement", "prenorm")
class PreNormBlock(Part):
    """h = x + mixer(norm(x)); y = h + ffn(norm(h))  (crates/hi-mlx/src/models.rs:6143-6149).

    The residual stream is float32. A sub-layer's output is carried as ``pending`` and added
    inside the next norm kernel, so each residual sum is one fused read-modify-write.
    """

    graph_safe = True

    def forward(self, layer, residual, pending, ctx, cache_view):
        h = layer.norm_mixer.forward(residual, pending)
        pending = layer.mixer.forward(h, ctx, cache_view)
        if getattr(layer.feed_forward, "wants_f32_input", False):
            h, h32 = layer.norm_feed_forward.forward(residual, pending, also_f32=True)
            pending = layer.feed_forward.forward(h, ctx, normed_f32=h32)
        else:
            h = layer.norm_feed_forward.forward(residual, pending)
            pending = layer.feed_forward.forward(h, ctx)
        return residual, pending

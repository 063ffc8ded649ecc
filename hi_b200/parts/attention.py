"""The attention mixer: grouped-query attention over a paged cache, global or windowed."""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .basic import Part
from .linear import linear
from .registry import build, register
from .spec import CacheSpec, PartSpec, TensorSpec


@register("mixer", "attention")
class AttentionMixer(Part):
    """q/k/v projections, position encoding or temperature, optional weightless q/k norm, cache
    append, softmax(q k^T scale + mask) v, output projection
    (Llama4Attention::forward, crates/hi-mlx/src/models.rs:5978-6052).

    params:
      ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``
      ``window``       None (every earlier key) | ("chunk", C) | ("sliding", W)
      ``position``     PartSpec of the position family
      ``qk_norm``, ``qk_norm_eps``   weightless L2 norm of q and k after the rotation
      ``temperature``  None | (floor_scale, attn_scale): q *= 1 + attn_scale*ln(1 + floor((pos+1)/floor_scale))
      ``scale``        softmax scale; default head_dim ** -0.5 (models.rs:5963)
      ``bias``         the random-weights writer makes ``<prefix>.{q,k,v,o}_proj.bias`` too
    tensors: ``<prefix>.{q,k,v,o}_proj.weight``, and each projection's ``.bias`` where the
    checkpoint has one (a bias is used iff its tensor exists: crates/hi-mlx/src/models.rs:1808,
    1843-1845).
    """

    graph_safe = True
    FUSED_DECODE = True      # decode steps: one launch for encoding, cache append, attention and merge

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        p = params
        self.hidden = int(p["hidden_size"])
        self.nh, self.nkv, self.hd = int(p["num_heads"]), int(p["num_kv_heads"]), int(p["head_dim"])
        if self.nh % self.nkv:
            raise ValueError(f"{prefix}: {self.nh} heads are not a multiple of {self.nkv} kv heads")
        if self.hd % 16 or self.hd > 256:
            raise ValueError(f"{prefix}: head_dim {self.hd} is not supported (multiples of 16 up to 256)")
        self.window = tuple(p["window"]) if p.get("window") else None
        self.position = build("position", p.get("position") or PartSpec("none"), env, prefix)
        self.qk_norm = bool(p.get("qk_norm", False))
        self.qk_norm_eps = float(p.get("qk_norm_eps", 1e-6))
        self.temperature = tuple(p["temperature"]) if p.get("temperature") else None
        self.scale = float(p.get("scale") or self.hd ** -0.5)
        self.bias = bool(p.get("bias", False))
        self.w_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None
        self.b_qkv: Optional[torch.Tensor] = None
        self.b_o: Optional[torch.Tensor] = None

    def cache_spec(self):
        return CacheSpec(kv_heads=self.nkv, head_dim=self.hd, window=self.window)

    def tensor_specs(self):
        h, nh, nkv, hd = self.hidden, self.nh, self.nkv, self.hd
        init = "normal" if self.bias else "absent"     # "absent": the random-weights writer leaves them out
        return [TensorSpec(f"{self.prefix}.q_proj.weight", (nh * hd, h)),
                TensorSpec(f"{self.prefix}.k_proj.weight", (nkv * hd, h)),
                TensorSpec(f"{self.prefix}.v_proj.weight", (nkv * hd, h)),
                TensorSpec(f"{self.prefix}.o_proj.weight", (h, nh * hd)),
                TensorSpec(f"{self.prefix}.q_proj.bias", (nh * hd,), init=init, optional=True),
                TensorSpec(f"{self.prefix}.k_proj.bias", (nkv * hd,), init=init, optional=True),
                TensorSpec(f"{self.prefix}.v_proj.bias", (nkv * hd,), init=init, optional=True),
                TensorSpec(f"{self.prefix}.o_proj.bias", (h,), init=init, optional=True)]

    def load(self, fetch):
        q, k, v = (fetch(f"{self.prefix}.{n}_proj.weight") for n in "qkv")
        if not (q.dtype == k.dtype == v.dtype):
            q, k, v = q.float(), k.float(), v.float()
        self.w_qkv = torch.cat([q, k, v], dim=0).contiguous()     # one product for q, k and v
        self.w_o = fetch(f"{self.prefix}.o_proj.weight").contiguous()
        biases = [fetch(f"{self.prefix}.{n}_proj.bias") for n in "qkv"]
        if any(b is not None for b in biases):          # a projection without one adds zeros
            sizes = (self.nh * self.hd, self.nkv * self.hd, self.nkv * self.hd)
            biases = [torch.zeros(n, dtype=self.w_qkv.dtype, device=self.w_qkv.device) if b is None else b
                      for b, n in zip(biases, sizes)]
            self.b_qkv = torch.cat([b.to(self.w_qkv.dtype) for b in biases]).contiguous()
        b_o = fetch(f"{self.prefix}.o_proj.bias")
        self.b_o = None if b_o is None else b_o.to(self.w_o.dtype).contiguous()

    def _key_splits(self, ctx, chunk: int, sliding: int, single: bool, device) -> int:
        """Portions far into long contexts on a layer that sees every key: all blocks of the
        tensor-core prefill kernel then have about the same many key tiles, and a partly filled
        last round of blocks is worth splitting the keys for (ops.prefill_key_splits)."""
        if chunk or sliding:
            return 1
        portions = [(s, n) for s, n in zip(ctx.start_pos, ctx.n_new) if n > 1 or not single]
        if not portions:
            return 1
        shortest, longest_new = min(s for s, _n in portions), max(n for _s, n in portions)
        if shortest < 2 * longest_new:
            return 1
        blocks = self.nh * sum(-(-n // ops.PREFILL_TC_MIN_TOKENS) for _s, n in portions)
        return ops.prefill_key_splits(blocks, shortest // 64, ops.sm_count(device))

    def forward(self, normed, ctx, cache):
        qkv = linear(normed, self.w_qkv, bias=self.b_qkv)
        positions = ctx.positions
        table = self.position.rotary_table()
        if table is None and hasattr(self.position, "apply"):
            # a position part without a rotary table encodes q and k itself
            n = qkv.shape[0]
            q, k, v = qkv.split([self.nh * self.hd, self.nkv * self.hd, self.nkv * self.hd], dim=1)
            q, k = self.position.apply(q.reshape(n, self.nh, self.hd), k.reshape(n, self.nkv, self.hd), positions)
            qkv = torch.cat([q.reshape(n, -1), k.reshape(n, -1), v], dim=1).to(normed.dtype).contiguous()
        inv_freq, interleaved = table if table is not None else (None, False)
        block_table = ctx.block_tables[cache.group]
        chunk = self.window[1] if self.window and self.window[0] == "chunk" else 0
        sliding = self.window[1] if self.window and self.window[0] == "sliding" else 0
        if ctx.max_new == 1 and cache.writes and self.FUSED_DECODE and qkv.dtype == torch.bfloat16:
            # a step of single decoded tokens: encoding, cache append, attention and the merge of its
            # splits in one launch, where the kernel takes the shapes
            o = ops.decode_attention_fused(qkv, self.nh, self.nkv, self.hd, positions, inv_freq, interleaved, self.qk_norm,
                                           self.qk_norm_eps, self.temperature, ctx.seq_of_token, block_table,
                                           cache.k_pages, cache.v_pages, chunk, sliding, self.scale, ctx.max_context)
            if o is not None:
                return linear(o.view(o.shape[0], self.nh * self.hd), self.w_o, bias=self.b_o)
        q = ops.qkv_post(qkv, self.nh, self.nkv, self.hd, positions, inv_freq, interleaved, self.qk_norm,
                         self.qk_norm_eps, self.temperature, ctx.seq_of_token, block_table, cache.k_pages,
                         cache.v_pages, ctx.page_size, cache.writes)
        if ctx.max_new == 1 and ops.decode_attention_supported(q.dtype, self.nh, self.nkv, self.hd):
            # every token of the step is one request's decoded token: the tensor-core kernel
            o = ops.decode_attention(q, cache.k_pages, cache.v_pages, block_table, ctx.seq_of_token, positions,
                                     chunk, sliding, self.scale, ctx.max_context)
        elif ctx.max_new > 1 and ops.prefill_attention_supported(q.dtype, self.nh, self.nkv, self.hd):
            # portions of prompts (single tokens of other requests ride along as one-row tiles)
            single = ctx.decode_rows is not None and ops.decode_attention_supported(q.dtype, self.nh, self.nkv, self.hd)
            # at least a tile of new tokens somewhere: the tcgen05 kernel; short portions: mma.sync
            tc = ctx.max_new >= ops.PREFILL_TC_MIN_TOKENS and ops.prefill_attention_tc_supported(
                q.dtype, self.nh, self.nkv, self.hd, ctx.page_size)
            if tc:
                o = ops.prefill_attention_tc(q, cache.k_pages, cache.v_pages, block_table, ctx.cu_seqlens, positions,
                                             ctx.n_seqs, ctx.max_new, chunk, sliding, self.scale, skip_single=single,
                                             key_splits=self._key_splits(ctx, chunk, sliding, single, q.device))
            else:
                o = ops.prefill_attention(q, cache.k_pages, cache.v_pages, block_table, ctx.cu_seqlens, positions,
                                          ctx.n_seqs, ctx.max_new, chunk, sliding, self.scale, skip_single=single)
            if single:
                # single tokens beside portions: their long key ranges go through the split decode kernel
                rows = ctx.decode_rows
                od = ops.decode_attention(q.index_select(0, rows), cache.k_pages, cache.v_pages, block_table,
                                          ctx.seq_of_token.index_select(0, rows), positions.index_select(0, rows),
                                          chunk, sliding, self.scale, ctx.decode_max_context)
                o.index_copy_(0, rows, od)
        else:
            o = ops.paged_attention(q, cache.k_pages, cache.v_pages, block_table, ctx.seq_of_token, positions,
                                    chunk, sliding, self.scale, ctx.max_context)
        return linear(o.view(o.shape[0], self.nh * self.hd), self.w_o, bias=self.b_o)

"""Typed configuration of the Llama 4 text decoder, read from config.json.

Key handling follows the reference parser (crates/hi-mlx/src/config.rs:305-521):
a nested ``text_config`` supplies the sizes and options, the top level keeps
``architectures`` / ``model_type``; ``eos_token_id`` may be an int or a list and is
merged with ``generation_config.json`` (config.rs:485-520, 809-823).

Keys the reference never reads (``attention_chunk_size``, ``attn_temperature_tuning``,
``floor_scale``, ``attn_scale``, ``interleave_moe_layer_step``, ``moe_layers``,
``intermediate_size_mlp``, ``nope_layer_interval``) are read here because the
architecture needs them; the reference hard-wires NoPE to every 4th layer
(crates/hi-mlx/src/models.rs:5953-5954) and MoE to every layer (models.rs:6105-6110).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, get_key as _get, read_config_files, token_ids as _token_ids


@dataclass(frozen=True)
class RopeScaling:
    """llama3 "NTK by parts" scaling; defaults as in models.rs:5898-5906."""

    factor: float = 8.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: float = 8192.0


@dataclass(frozen=True)
class Llama4TextConfig:
    # sizes
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    # norms
    rms_norm_eps: float
    # positions
    rope_theta: float
    rope_scaling: Optional[RopeScaling]
    rope_interleaved: bool
    rope_layers: Tuple[bool, ...]          # per layer: True = rotary, False = NoPE (global)
    # attention options
    attention_chunk_size: int
    use_qk_norm: bool
    qk_norm_eps: float
    attn_temperature_tuning: bool
    floor_scale: float
    attn_scale: float
    attention_bias: bool
    # feed-forward
    moe_layers: Tuple[bool, ...]           # per layer: True = experts, False = dense SwiGLU
    num_local_experts: int
    num_experts_per_tok: int
    intermediate_size: int                 # each expert and the shared expert
    intermediate_size_mlp: int             # dense layers
    hidden_act: str
    # head and bookkeeping
    tie_word_embeddings: bool
    max_position_embeddings: Optional[int]
    eos_token_ids: Tuple[int, ...]
    bos_token_id: Optional[int]
    pad_token_id: Optional[int]
    torch_dtype: Optional[str]
    architectures: Tuple[str, ...]
    model_type: str
    raw: Dict[str, Any] = field(repr=False, compare=False, default_factory=dict)

    @staticmethod
    def from_json(raw: Dict[str, Any], generation_config: Optional[Dict[str, Any]] = None) -> "Llama4TextConfig":
        if not isinstance(raw, dict):
            raise ConfigError("config.json: top level must be an object")
        top = raw
        text = raw.get("text_config") if isinstance(raw.get("text_config"), dict) else None
        src = dict(text) if text is not None else dict(raw)
        if text is not None:
            # sizes come from text_config; keys it lacks fall back to the top level
            for k, v in top.items():
                src.setdefault(k, v)

        hidden = _get(src, "hidden_size", int, required=True)
        heads = _get(src, "num_attention_heads", int, required=True)
        vocab = _get(src, "vocab_size", int, required=True)
        layers = _get(src, "num_hidden_layers", int, required=True)
        for key, v in (("hidden_size", hidden), ("num_attention_heads", heads),
                       ("vocab_size", vocab), ("num_hidden_layers", layers)):
            if v <= 0:
                raise ConfigError(f"config.json: '{key}' must be positive, got {v}")
        kv_heads = _get(src, "num_key_value_heads", int, default=heads)
        if kv_heads <= 0 or heads % kv_heads != 0:
            raise ConfigError(
                f"config.json: 'num_attention_heads' ({heads}) must be a multiple of "
                f"'num_key_value_heads' ({kv_heads})")
        head_dim = _get(src, "head_dim", int, default=None)
        if head_dim is None:
            if hidden % heads != 0:
                raise ConfigError(
                    f"config.json: 'head_dim' is absent and 'hidden_size' ({hidden}) is not a "
                    f"multiple of 'num_attention_heads' ({heads})")
            head_dim = hidden // heads
        if head_dim <= 0 or head_dim % 2 != 0:
            raise ConfigError(f"config.json: 'head_dim' must be a positive even number, got {head_dim}")

        eps = _get(src, "rms_norm_eps", float, default=1e-6)          # config.rs:424
        theta = _get(src, "rope_theta", float, default=1_000_000.0)  # config.rs:425-433
        if theta <= 0:
            raise ConfigError(f"config.json: 'rope_theta' must be positive, got {theta}")
        scaling = None
        rs = src.get("rope_scaling")
        if rs is not None:
            if not isinstance(rs, dict):
                raise ConfigError("config.json: 'rope_scaling' must be an object or null")
            kind = rs.get("rope_type", rs.get("type", "llama3"))
            if kind not in ("llama3",):
                raise ConfigError(f"config.json: rope_scaling type {kind!r} is not supported (llama3 only)")
            d = RopeScaling()
            scaling = RopeScaling(
                factor=_get(rs, "factor", float, d.factor),
                low_freq_factor=_get(rs, "low_freq_factor", float, d.low_freq_factor),
                high_freq_factor=_get(rs, "high_freq_factor", float, d.high_freq_factor),
                original_max_position_embeddings=_get(
                    rs, "original_max_position_embeddings", float, d.original_max_position_embeddings),
            )
            if scaling.factor <= 0 or scaling.low_freq_factor <= 0 or scaling.high_freq_factor <= 0:
                raise ConfigError("config.json: 'rope_scaling' factors must be positive")

        # which layers rotate: an explicit list wins (1 = rotary, 0 = NoPE), else the interval
        no_rope = src.get("no_rope_layers")
        if isinstance(no_rope, list) and len(no_rope) > 0:
            if len(no_rope) != layers:
                raise ConfigError(
                    f"config.json: 'no_rope_layers' has {len(no_rope)} entries for {layers} layers")
            rope_layers = tuple(bool(int(v)) for v in no_rope)
        else:
            interval = _get(src, "nope_layer_interval", int, default=4)
            if interval < 0:
                raise ConfigError(f"config.json: 'nope_layer_interval' must be >= 0, got {interval}")
            rope_layers = tuple(not (interval > 0 and (i + 1) % interval == 0) for i in range(layers))

        chunk = _get(src, "attention_chunk_size", int, default=8192)
        if chunk <= 0:
            raise ConfigError(f"config.json: 'attention_chunk_size' must be positive, got {chunk}")
        floor_scale = _get(src, "floor_scale", float, default=8192.0)
        if floor_scale <= 0:
            raise ConfigError(f"config.json: 'floor_scale' must be positive, got {floor_scale}")

        experts = _get(src, "num_local_experts", int, default=0)
        top_k = _get(src, "num_experts_per_tok", int, default=1)
        moe_list = src.get("moe_layers")
        if isinstance(moe_list, list) and len(moe_list) > 0:
            bad = [i for i in moe_list if not isinstance(i, int) or i < 0 or i >= layers]
            if bad:
                raise ConfigError(f"config.json: 'moe_layers' names layers {bad} outside 0..{layers - 1}")
            moe_layers = tuple(i in set(moe_list) for i in range(layers))
        else:
            step = _get(src, "interleave_moe_layer_step", int, default=1)
            if step < 0:
                raise ConfigError(f"config.json: 'interleave_moe_layer_step' must be >= 0, got {step}")
            moe_layers = tuple(step > 0 and (i + 1) % step == 0 for i in range(layers))
        inter = _get(src, "intermediate_size", int, default=0)
        inter_mlp = _get(src, "intermediate_size_mlp", int, default=0)
        if any(moe_layers):
            if experts <= 0:
                raise ConfigError("config.json: layers with experts need 'num_local_experts' > 0")
            if top_k <= 0 or top_k > experts:
                raise ConfigError(
                    f"config.json: 'num_experts_per_tok' ({top_k}) must lie in 1..num_local_experts ({experts})")
            if inter <= 0:
                raise ConfigError("config.json: layers with experts need 'intermediate_size' > 0")
        if not all(moe_layers) and inter_mlp <= 0:
            raise ConfigError("config.json: dense layers need 'intermediate_size_mlp' > 0")
        act = src.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: 'hidden_act' {act!r} is not supported (silu only)")

        eos = _token_ids(src, "eos_token_id")
        if generation_config:
            for t in _token_ids(generation_config, "eos_token_id"):
                if t not in eos:
                    eos.append(t)
        max_pos = _get(src, "max_position_embeddings", int, default=None)
        archs = top.get("architectures") or src.get("architectures") or []
        if isinstance(archs, str):
            archs = [archs]
        return Llama4TextConfig(
            vocab_size=vocab, hidden_size=hidden, num_hidden_layers=layers,
            num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim,
            rms_norm_eps=eps, rope_theta=theta, rope_scaling=scaling,
            rope_interleaved=_get(src, "rope_interleaved", bool, default=False),
            rope_layers=rope_layers, attention_chunk_size=chunk,
            use_qk_norm=_get(src, "use_qk_norm", bool, default=False),       # models.rs:5966-5971
            qk_norm_eps=_get(src, "qk_norm_eps", float, default=1e-6),      # models.rs:6019-6020
            attn_temperature_tuning=_get(src, "attn_temperature_tuning", bool, default=False),
            floor_scale=floor_scale, attn_scale=_get(src, "attn_scale", float, default=0.1),
            attention_bias=_get(src, "attention_bias", bool, default=False),
            moe_layers=moe_layers, num_local_experts=experts, num_experts_per_tok=top_k,
            intermediate_size=inter, intermediate_size_mlp=inter_mlp, hidden_act=act,
            tie_word_embeddings=_get(src, "tie_word_embeddings", bool, default=False),
            max_position_embeddings=max_pos, eos_token_ids=tuple(eos),
            bos_token_id=_get(src, "bos_token_id", int, default=None) if not isinstance(src.get("bos_token_id"), list) else None,
            pad_token_id=_get(src, "pad_token_id", int, default=None),
            torch_dtype=src.get("torch_dtype") if isinstance(src.get("torch_dtype"), str) else None,
            architectures=tuple(str(a) for a in archs),
            model_type=str(top.get("model_type") or src.get("model_type") or ""),
            raw=raw,
        )

    @staticmethod
    def from_dir(model_dir: str) -> "Llama4TextConfig":
        return Llama4TextConfig.from_json(*read_config_files(model_dir))

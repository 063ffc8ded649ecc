"""The Llama 4 text decoder as data: its configuration turned into a ModelSpec.

Layer kinds (crates/hi-mlx/src/models.rs:5893-6230 for the Scout subset the reference runs;
chunked attention, attention temperature, dense layers and top-k > 1 are read from the
configuration keys the reference ignores):
  rotary layers  attention within blocks of ``attention_chunk_size`` positions, llama3-scaled
                 rotation, optional weightless q/k norm;
  NoPE layers    attention over every earlier token, no rotation, optional temperature on q;
  feed-forward   sigmoid-routed top-k experts with a shared expert, or dense SwiGLU.
"""
from __future__ import annotations

from dataclasses import asdict
from typing import Optional

from ..config.llama4 import ConfigError, Llama4TextConfig
from .spec import LayerSpec, ModelSpec, PartSpec


def build_llama4_spec(cfg: Llama4TextConfig) -> ModelSpec:
    if cfg.head_dim % 16 != 0 or cfg.head_dim > 256:
        raise ConfigError(f"config.json: 'head_dim' {cfg.head_dim} is not supported (multiples of 16 up to 256)")
    scaling = asdict(cfg.rope_scaling) if cfg.rope_scaling else None
    rope = PartSpec("rope", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta, "scaling": scaling,
                             "interleaved": cfg.rope_interleaved})
    layers = []
    for i in range(cfg.num_hidden_layers):
        rotary = cfg.rope_layers[i]
        mixer = PartSpec("attention", {
            "name": "self_attn", "hidden_size": cfg.hidden_size, "num_heads": cfg.num_attention_heads,
            "num_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "window": ("chunk", cfg.attention_chunk_size) if rotary else None,
            "position": rope if rotary else PartSpec("none"),
            "qk_norm": cfg.use_qk_norm and rotary, "qk_norm_eps": cfg.qk_norm_eps,
            "temperature": (cfg.floor_scale, cfg.attn_scale) if (cfg.attn_temperature_tuning and not rotary) else None,
            "bias": cfg.attention_bias,
        })
        if cfg.moe_layers[i]:
            ffn = PartSpec("moe_sigmoid", {
                "name": "feed_forward", "hidden_size": cfg.hidden_size, "num_experts": cfg.num_local_experts,
                "top_k": cfg.num_experts_per_tok, "intermediate_size": cfg.intermediate_size, "shared_expert": True})
        else:
            ffn = PartSpec("dense_swiglu", {"name": "feed_forward", "hidden_size": cfg.hidden_size,
                                            "intermediate_size": cfg.intermediate_size_mlp})
        norm = lambda name: PartSpec("rmsnorm", {"name": name, "size": cfg.hidden_size, "eps": cfg.rms_norm_eps})
        layers.append(LayerSpec(prefix=f"model.layers.{i}", mixer=mixer, feed_forward=ffn,
                                norm_mixer=norm("input_layernorm"), norm_feed_forward=norm("post_attention_layernorm"),
                                arrangement="prenorm"))
    return ModelSpec(
        hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size,
        embedding=PartSpec("token_embedding", {"name": "model.embed_tokens", "vocab_size": cfg.vocab_size,
                                               "hidden_size": cfg.hidden_size}),
        layers=tuple(layers), schedule=ModelSpec.sequential(cfg.num_hidden_layers),
        final_norm=PartSpec("rmsnorm", {"name": "model.norm", "size": cfg.hidden_size, "eps": cfg.rms_norm_eps}),
        head=PartSpec("linear_head", {"name": "lm_head", "vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
                                      "tie": cfg.tie_word_embeddings}),
        eos_token_ids=cfg.eos_token_ids, max_position_embeddings=cfg.max_position_embeddings)


def normalize_llama4_tensor_name(name: str) -> Optional[str]:
    """Strip ``language_model.`` (leading, or after ``model.``) and drop what is not the text
    decoder: vision tower, projector, multi-token-prediction heads
    (crates/hi-mlx/src/weights.rs:456-482)."""
    if name.startswith("language_model."):
        name = name[len("language_model."):]
    elif name.startswith("model.language_model."):
        name = "model." + name[len("model.language_model."):]
    if name.startswith(("visual.", "vision_", "vision_model.", "multi_modal_projector.", "mtp.")) or ".mtp." in name:
        return None
    if name.startswith(("model.", "lm_head.")):
        return name
    return None


def derive_llama4_tensors(shapes):
    """The routed experts of a checkpoint in the original export layout, one fused tensor per layer
    with the input dimension first and no ``.weight`` suffix: ``experts.gate_up_proj`` [E, H, 2I]
    (gate columns, then up) and ``experts.down_proj`` [E, I, H]. The parts ask for the converted
    layout the reference reads, ``experts.{gate,up}_proj.weight`` [E, I, H] and
    ``experts.down_proj.weight`` [E, H, I] (crates/hi-mlx/src/models.rs:6070, 3138-3166); they are
    cut and transposed here, on the device."""
    from ..weights.loader import DerivedTensor

    out = {}
    for name, shape in shapes.items():
        if name.endswith(".experts.gate_up_proj") and len(shape) == 3 and shape[2] % 2 == 0:
            base = name[: -len("gate_up_proj")]
            e, h, two_i = shape
            half = two_i // 2
            out[base + "gate_proj.weight"] = DerivedTensor(
                [name], (e, half, h), lambda ts, half=half: ts[0][:, :, :half].transpose(1, 2).contiguous())
            out[base + "up_proj.weight"] = DerivedTensor(
                [name], (e, half, h), lambda ts, half=half: ts[0][:, :, half:].transpose(1, 2).contiguous())
        elif name.endswith(".experts.down_proj") and len(shape) == 3:
            e, i, h = shape
            out[name + ".weight"] = DerivedTensor([name], (e, h, i), lambda ts: ts[0].transpose(1, 2).contiguous())
    return out

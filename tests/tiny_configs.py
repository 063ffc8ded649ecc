"""The two tiny Llama 4 configurations of the tests; they differ in every size and option."""

TINY_A = {
    "architectures": ["Llama4ForCausalLM"], "model_type": "llama4_text",
    "vocab_size": 256, "hidden_size": 64, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "rope_scaling": None,
    "attention_chunk_size": 32, "nope_layer_interval": 2,
    "use_qk_norm": True, "attn_temperature_tuning": True, "floor_scale": 16, "attn_scale": 0.1,
    "interleave_moe_layer_step": 1, "num_local_experts": 4, "num_experts_per_tok": 1,
    "intermediate_size": 128, "intermediate_size_mlp": 256,
    "tie_word_embeddings": False, "max_position_embeddings": 4096, "eos_token_id": 2,
}

# nested like a multimodal checkpoint's config: sizes under text_config
TINY_B = {
    "architectures": ["Llama4ForConditionalGeneration"], "model_type": "llama4",
    "text_config": {
        "model_type": "llama4_text",
        "vocab_size": 515, "hidden_size": 192, "num_hidden_layers": 6,
        "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 32,
        "rms_norm_eps": 1e-6, "rope_theta": 500000.0,
        "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                         "original_max_position_embeddings": 64},
        "attention_chunk_size": 16, "nope_layer_interval": 4,
        "use_qk_norm": False, "attn_temperature_tuning": False,
        "interleave_moe_layer_step": 2, "num_local_experts": 8, "num_experts_per_tok": 2,
        "intermediate_size": 96, "intermediate_size_mlp": 384,
        "tie_word_embeddings": True, "max_position_embeddings": 2048, "eos_token_id": [1, 7],
    },
}

# a third shape for kernels and parts: 5 query heads per kv head, head_dim 48, odd widths, biases on q/k/v/o
TINY_C = {
    "architectures": ["Llama4ForCausalLM"], "model_type": "llama4_text",
    "vocab_size": 331, "hidden_size": 120, "num_hidden_layers": 3,
    "num_attention_heads": 10, "num_key_value_heads": 2, "head_dim": 48,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 16.0, "low_freq_factor": 1.0, "high_freq_factor": 1.0,
                     "original_max_position_embeddings": 32},
    "attention_chunk_size": 24, "no_rope_layers": [1, 0, 1], "rope_interleaved": True, "attention_bias": True,
    "use_qk_norm": True, "attn_temperature_tuning": True, "floor_scale": 8, "attn_scale": 0.25,
    "moe_layers": [0, 2], "num_local_experts": 5, "num_experts_per_tok": 3,
    "intermediate_size": 72, "intermediate_size_mlp": 200,
    "tie_word_embeddings": False, "max_position_embeddings": 1024,
}

# head_dim 64 with 4 query heads per kv head: the shapes the tensor-core attention kernels take
TINY_D = {
    "architectures": ["Llama4ForCausalLM"], "model_type": "llama4_text",
    "vocab_size": 300, "hidden_size": 128, "num_hidden_layers": 3,
    "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 64,
    "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "rope_scaling": None,
    "attention_chunk_size": 48, "nope_layer_interval": 3,
    "use_qk_norm": True, "attn_temperature_tuning": True, "floor_scale": 32, "attn_scale": 0.1,
    "interleave_moe_layer_step": 1, "num_local_experts": 4, "num_experts_per_tok": 2,
    "intermediate_size": 64, "intermediate_size_mlp": 128,
    "tie_word_embeddings": False, "max_position_embeddings": 4096,
}

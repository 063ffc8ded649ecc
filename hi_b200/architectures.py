"""The architectures this package brings. Importing this module registers them; another
architecture is added the same way from anywhere: a typed config reader, a builder of a
:class:`~hi_b200.parts.spec.ModelSpec` and a tensor-name normaliser, handed to
:func:`~hi_b200.config.registry.register_architecture` under its ``architectures`` /
``model_type`` names (the reference routes ``llama4`` / ``llama4_text`` to its Llama 4 model:
crates/hi-mlx/src/config.rs:620-637, crates/hi-mlx/src/models.rs:373-375)."""
from .config.llama4 import Llama4TextConfig
from .config.registry import Architecture, register_architecture
from .parts.llama4 import build_llama4_spec, derive_llama4_tensors, normalize_llama4_tensor_name

register_architecture(
    ["Llama4ForConditionalGeneration", "Llama4ForCausalLM", "llama4", "llama4_text"],
    Architecture(name="llama4_text", parse_config=Llama4TextConfig.from_json, build_spec=build_llama4_spec,
                 normalize_tensor_name=normalize_llama4_tensor_name, derive_tensors=derive_llama4_tensors))

from .base import ConfigError
from .llama4 import Llama4TextConfig, RopeScaling
from .registry import Architecture, load_architecture, lookup, register_architecture, registered_architectures

__all__ = ["ConfigError", "Llama4TextConfig", "RopeScaling", "Architecture", "load_architecture", "lookup",
           "register_architecture", "registered_architectures"]

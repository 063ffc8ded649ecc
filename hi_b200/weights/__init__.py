from .loader import DerivedTensor, WeightError, check_names, load_from_dir, load_random, random_tensor, write_random_model
from .safetensors_io import Checkpoint, SafetensorsError, write_safetensors

__all__ = ["DerivedTensor", "WeightError", "check_names", "load_from_dir", "load_random", "random_tensor", "write_random_model",
           "Checkpoint", "SafetensorsError", "write_safetensors"]

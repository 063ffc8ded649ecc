"""hi_b200: a small, whole decoder inference engine for one B200 GPU; the architecture it brings
is the Llama 4 text decoder (``hi_b200/architectures.py``)."""
from .engine import LLM, Engine, GenerationOutput, StepEntry, generate
from .sampling import SamplingParams

__all__ = ["LLM", "Engine", "GenerationOutput", "StepEntry", "generate", "SamplingParams"]
__version__ = "0.1.0"

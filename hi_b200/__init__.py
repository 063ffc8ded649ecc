"""hi_b200: a small, whole Llama 4 text-decoder inference engine for one B200 GPU."""
from .engine import LLM, Engine, GenerationOutput, StepEntry, generate
from .sampling import SamplingParams

__all__ = ["LLM", "Engine", "GenerationOutput", "StepEntry", "generate", "SamplingParams"]
__version__ = "0.1.0"

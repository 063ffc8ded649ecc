from .core import Engine, EngineStats, StepEntry, parse_dtype
from .generate import LLM, GenerationOutput, generate
from .scheduler import PlannedEntry, Request, Scheduler, SchedulerConfig, StepPlan

__all__ = ["Engine", "EngineStats", "StepEntry", "parse_dtype", "LLM", "GenerationOutput", "generate",
           "PlannedEntry", "Request", "Scheduler", "SchedulerConfig", "StepPlan"]

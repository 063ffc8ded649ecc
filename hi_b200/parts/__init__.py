from .context import CacheView, Pending, StepContext
from .registry import BuildEnv, build, register, registered, unregister
from .spec import CacheSpec, LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSpec

__all__ = ["CacheView", "Pending", "StepContext", "BuildEnv", "build", "register", "registered", "unregister",
           "CacheSpec", "LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry", "TensorSpec"]

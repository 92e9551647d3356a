"""Engine: batch descriptor, the step function, the scheduler and the Python entry point."""

from .batch import BatchBuilder, StepBatch, StepEntry
from .engine import Engine, resolve_dtype

__all__ = ["BatchBuilder", "StepBatch", "StepEntry", "Engine", "resolve_dtype"]

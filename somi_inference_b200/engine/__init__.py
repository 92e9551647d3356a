"""Engine: batch descriptor, the step function, the scheduler and the Python entry point."""

from .batch import BatchBuilder, StepBatch, StepEntry
from .engine import Engine, resolve_dtype
from .llm import LLM
from .scheduler import Request, RequestStatus, ScheduledBatch, ScheduledItem, Scheduler

__all__ = ["BatchBuilder", "StepBatch", "StepEntry", "Engine", "resolve_dtype", "LLM", "Request",
           "RequestStatus", "ScheduledBatch", "ScheduledItem", "Scheduler"]

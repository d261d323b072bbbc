"""The engine: the step function over a model and its cache, and the scheduler above it."""
from .step import Engine, StepEntry, StepError

__all__ = ["Engine", "StepEntry", "StepError"]

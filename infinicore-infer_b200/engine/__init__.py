"""The engine: the step function over a model and its cache, the scheduler and the generation loop."""
from .scheduler import FINISHED, RUNNING, WAITING, Request, Scheduled, Scheduler
from .step import Engine, StepEntry, StepError
from .generator import Generator

__all__ = ["Engine", "StepEntry", "StepError", "Scheduler", "Request", "Scheduled", "Generator",
           "WAITING", "RUNNING", "FINISHED"]

"""The step function, the scheduler above it, and the request API."""

from .batch import StepContext, StepEntry
from .engine import Engine
from .request import Request
from .runner import ModelRunner
from .scheduler import Scheduler

__all__ = ["Engine", "ModelRunner", "Request", "Scheduler", "StepContext", "StepEntry"]

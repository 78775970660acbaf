from .context import KVView, StateView, StepContext
from .engine import Engine, RequestOutput
from .scheduler import Request, Scheduled, Scheduler
from .step import StepEntry, Stepper

__all__ = ["Engine", "KVView", "Request", "RequestOutput", "Scheduled", "Scheduler", "StateView", "StepContext",
           "StepEntry", "Stepper"]

from .context import KVView, StateView, StepContext
from .step import StepEntry, Stepper

__all__ = ["KVView", "StateView", "StepContext", "StepEntry", "Stepper"]

from .batch import StepContext, StepItem
from .core import Engine, StepError

__all__ = ["StepContext", "StepItem", "Engine", "StepError"]

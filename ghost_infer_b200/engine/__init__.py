from .model import Model
from .step import Engine, StepContext, StepEntry

__all__ = ["Model", "Engine", "StepContext", "StepEntry"]

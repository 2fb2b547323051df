"""The engine: step function, scheduler, generation loop."""

from .loading import load_model, random_model
from .step import StepContext, StepEntry, StepRunner

__all__ = ["StepEntry", "StepContext", "StepRunner", "load_model", "random_model"]

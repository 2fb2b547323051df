"""The engine: step function, scheduler, generation loop, Python entry point."""

from .engine import Engine
from .llm import LLM
from .loading import load_model, random_model
from .request import GenerationResult, Request, StopCriteria
from .scheduler import RequestRefused, Scheduler
from .step import StepContext, StepEntry, StepRunner

__all__ = ["Engine", "LLM", "Request", "StopCriteria", "GenerationResult", "Scheduler", "RequestRefused",
           "StepEntry", "StepContext", "StepRunner", "load_model", "random_model"]

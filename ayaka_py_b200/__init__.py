"""ayaka_py_b200: a single-GPU inference engine for GPT-2 on NVIDIA B200
(sm_100a), built after the Python/Triton engine gityuko-hb/ayaka-py."""

__version__ = "0.1.0"

from . import models, parts  # noqa: F401  (register architectures and part kinds)
from .config import EngineConfig, GPT2Config
from .engine import LLM, Request, StopCriteria
from .sampling import SamplingParams

__all__ = ["LLM", "Request", "StopCriteria", "SamplingParams", "EngineConfig", "GPT2Config", "__version__"]

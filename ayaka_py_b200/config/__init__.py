"""Typed configurations: one per architecture (read from its own config.json
keys) and one for the engine."""

from .model import ConfigError, GPT2Config, ModelConfig
from .engine import EngineConfig

__all__ = ["ConfigError", "ModelConfig", "GPT2Config", "EngineConfig"]

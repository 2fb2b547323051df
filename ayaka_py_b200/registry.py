"""One registry from an architecture's name (``config.json["architectures"][0]``)
to its configuration class and the function that writes its ``ModelSpec``.

The reference has no registry: its command line is an if/elif chain on
``model_type`` (``commands/cli.py:97-131``)."""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Callable

from .config.model import ConfigError, ModelConfig
from .parts.base import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str                                        # e.g. "GPT2LMHeadModel"
    model_type: str                                  # e.g. "gpt2", the fallback key
    config_class: type[ModelConfig]
    build_spec: Callable[[ModelConfig], ModelSpec]
    # checkpoint name -> canonical name, or None for a tensor to be ignored
    normalize_name: Callable[[str, ModelConfig], str | None] = lambda name, config: name


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(arch: Architecture) -> None:
    _ARCHITECTURES[arch.name] = arch


def registered_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def architecture_for(document: dict) -> Architecture:
    """Chosen by ``architectures[0]``; by ``model_type`` if that key is absent."""
    names = document.get("architectures") or []
    if names:
        if names[0] in _ARCHITECTURES:
            return _ARCHITECTURES[names[0]]
        raise ConfigError(f"unknown architecture {names[0]!r}; registered: {registered_architectures()}")
    model_type = document.get("model_type")
    for arch in _ARCHITECTURES.values():
        if arch.model_type == model_type:
            return arch
    raise ConfigError(
        f"config.json names no registered architecture (model_type {model_type!r}); "
        f"registered: {registered_architectures()}")


def read_config(folder) -> tuple[Architecture, ModelConfig]:
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{folder} does not contain config.json")
    document = json.loads(path.read_text(encoding="utf-8"))
    arch = architecture_for(document)
    return arch, arch.config_class.from_dict(document)

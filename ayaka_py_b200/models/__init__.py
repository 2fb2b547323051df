"""Architectures.  Importing this package registers them."""

from . import gpt2  # noqa: F401
from .model import Model

__all__ = ["Model"]

"""Weights: safetensors files, binding by name, the random-weights mode."""

from .loader import DictStore, FolderStore, WeightMismatchError, load_weights
from .random_init import random_tensors, write_random_model
from .safetensors import (CheckpointCorruptError, SafetensorsFile, UnsupportedWeightFormatError,
                          write_safetensors)

__all__ = ["CheckpointCorruptError", "UnsupportedWeightFormatError", "SafetensorsFile", "write_safetensors", "WeightMismatchError",
           "FolderStore", "DictStore", "load_weights", "random_tensors", "write_random_model"]

"""Sampling: options, seed rule and the sampler that calls the kernel."""

from .params import SamplingParams, derive_seed, splitmix64
from .sampler import Sampler

__all__ = ["SamplingParams", "Sampler", "derive_seed", "splitmix64"]

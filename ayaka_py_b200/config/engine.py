"""Engine options: cache geometry, batch limits and precision.

Names follow the reference's command line where it has them
(``commands/cli.py:25-37``): ``kv_pages``, ``page_size``, ``max_requests``,
``batch_tokens``, ``prefill_chunk``, ``max_model_len``, ``decode_graph``."""

from __future__ import annotations

from dataclasses import dataclass

from .model import ConfigError

_DTYPES = {"float32": "float32", "fp32": "float32", "bfloat16": "bfloat16", "bf16": "bfloat16"}


@dataclass(frozen=True)
class EngineConfig:
    dtype: str = "bfloat16"
    kv_pages: int = 1024          # pages per cache group, the padding page included
    kv_cache_bytes: int | None = None   # instead of kv_pages: one byte budget, split over the groups by what a page of each costs
    page_size: int = 16           # tokens in a page
    max_requests: int = 32        # live requests = state slots
    batch_tokens: int = 256       # token budget of one step
    prefill_chunk: int = 128      # largest portion of one prompt in a step
    max_model_len: int | None = None   # None: the model's own limit
    decode_graph: bool = True     # replay pure-decode steps from CUDA graphs (False: every kernel launched from Python)
    lookahead: bool = True        # plan and launch the next step while this one's tokens are on their way
    seed: int = 0                 # base of the seeds of requests that name none

    def __post_init__(self) -> None:
        if self.dtype not in _DTYPES:
            raise ConfigError(f"dtype must be one of {sorted(set(_DTYPES))}, got {self.dtype!r}")
        object.__setattr__(self, "dtype", _DTYPES[self.dtype])
        for name in ("kv_pages", "page_size", "max_requests", "batch_tokens", "prefill_chunk"):
            value = getattr(self, name)
            if isinstance(value, bool) or not isinstance(value, int) or value < 1:
                raise ConfigError(f"{name} must be a positive integer, got {value!r}")
        if self.page_size & (self.page_size - 1):
            raise ConfigError(f"page_size must be a power of two, got {self.page_size}")
        if self.kv_pages < 2:
            raise ConfigError("kv_pages must be at least 2 (one page is the padding page)")
        if self.kv_cache_bytes is not None and (isinstance(self.kv_cache_bytes, bool) or not isinstance(self.kv_cache_bytes, int)
                                                or self.kv_cache_bytes < 1):
            raise ConfigError(f"kv_cache_bytes must be a positive integer or None, got {self.kv_cache_bytes!r}")
        if self.max_model_len is not None and self.max_model_len < 1:
            raise ConfigError("max_model_len must be positive")

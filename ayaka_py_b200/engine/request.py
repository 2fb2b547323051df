"""Requests as the engine sees them (``request/schema.py:14-102``)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

from ..sampling.params import SamplingParams


@dataclass(frozen=True)
class StopCriteria:
    max_tokens: int = 128
    min_tokens: int = 0
    stop_token_ids: tuple[int, ...] = ()
    ignore_eos: bool = False

    def __post_init__(self) -> None:
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be at least 1")
        if not 0 <= self.min_tokens <= self.max_tokens:
            raise ValueError("min_tokens must be in [0, max_tokens]")


@dataclass(frozen=True)
class Request:
    request_id: str
    prompt_token_ids: Sequence[int]
    sampling: SamplingParams = SamplingParams()
    stop: StopCriteria = StopCriteria()

    def __post_init__(self) -> None:
        if len(self.prompt_token_ids) == 0:
            raise ValueError("a request needs at least one prompt token")     # request/schema.py:91-92

    @property
    def max_total_len(self) -> int:
        return len(self.prompt_token_ids) + self.stop.max_tokens


@dataclass
class GenerationResult:
    request_id: str
    prompt_token_ids: list[int]
    token_ids: list[int] = field(default_factory=list)
    finish_reason: str | None = None      # "stop", "eos", "length", "abort"
    preemptions: int = 0

"""Sampling options of a request, with the reference's names and defaults
(``sampling/params.py:24-134``), and the seed rule for requests that name none
(``sampling/rng.py:220-267``)."""

from __future__ import annotations

from dataclasses import dataclass

_MASK64 = 0xFFFFFFFFFFFFFFFF


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 1.0      # 0: greedy
    top_k: int = -1               # <= 0: off; 1: greedy
    top_p: float = 1.0
    min_p: float = 0.0
    seed: int | None = None       # None: derived from the request's admission ordinal

    def __post_init__(self) -> None:
        if not self.temperature >= 0.0:
            raise ValueError("temperature must be >= 0")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")
        if not 0.0 <= self.min_p <= 1.0:
            raise ValueError("min_p must be in [0, 1]")
        if isinstance(self.top_k, bool) or not isinstance(self.top_k, int):
            raise ValueError("top_k must be an integer")
        if self.seed is not None and not 0 <= self.seed < 1 << 63:
            raise ValueError("seed must be in [0, 2**63)")

    @property
    def greedy(self) -> bool:
        """``temperature == 0 or top_k == 1`` (``sampling/params.py:127-134``)."""
        return self.temperature == 0.0 or self.top_k == 1

    @property
    def filtered(self) -> bool:
        return self.top_k > 1 or self.top_p < 1.0 or self.min_p > 0.0


def splitmix64(x: int) -> int:
    z = (x + 0x9E3779B97F4A7C15) & _MASK64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK64
    return z ^ (z >> 31)


def derive_seed(request_index: int) -> int:
    """Seed of a request that names none: splitmix64 of its admission ordinal,
    kept below 2**63."""
    return splitmix64(request_index) & 0x7FFFFFFFFFFFFFFF

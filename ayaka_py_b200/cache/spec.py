"""Data that the model and the cache manager share."""

from __future__ import annotations

from dataclasses import dataclass

from ..parts.base import KVNeed, StateNeed


@dataclass(frozen=True)
class CacheGroupSpec:
    """Run steps with the same need: one namespace of pages and one block table
    per request (KV), or one region of state slots (state)."""
    name: str
    need: KVNeed | StateNeed
    layers: int                     # run steps that keep a cache of their own in this group


@dataclass(frozen=True)
class CacheBinding:
    """What a run step's mixer gets: its group and its index among the group's
    layers.  ``writes`` is False for a run step that reads another's cache."""
    group: int
    name: str
    layer: int
    writes: bool = True

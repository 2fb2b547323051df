"""What a part is, and the registries that the model is built from.

A model is put together from parts: an embedding, a position encoding, and for
every layer a norm, a mixer (attention here), a second norm and a feed-forward,
arranged by a block; then a final norm and a head.  Each part

* is made from plain parameters (sizes and constants), never from a model
  configuration, and does not know which model it is in;
* declares the tensors it holds (``tensors()``), in its own layout;
* gets them bound after loading (``bind``);
* and, when it keeps something per request, declares what it needs from the
  cache manager (``cache_need``).

An architecture only writes a ``ModelSpec``: which part kinds with which
parameters in which layer, where each tensor comes from in the checkpoint, and
the order in which the layers run.  New kinds are added with ``register_part``;
nothing else in the package changes.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, ClassVar

import torch


# ----------------------------------------------------------------- tensors --

@dataclass(frozen=True)
class Init:
    """Distribution of a tensor in the random-weights mode: mean + std * N(0,1)."""
    std: float = 0.02
    mean: float = 0.0


@dataclass(frozen=True)
class TensorDecl:
    """A tensor as the part holds it.

    kind ``matrix``: a GEMM operand or table, kept in the compute dtype
    (bfloat16 or float32); ``vector``: small parameters used in 32-bit
    arithmetic (norm weights, biases), kept in float32; ``int``: integer
    tables, kept in int32."""
    shape: tuple[int, ...]
    kind: str = "matrix"


@dataclass(frozen=True)
class Source:
    """Where a part's tensor comes from in the checkpoint.

    ``transposed``: the checkpoint stores the transpose of the part's layout
    (GPT-2's Conv1D weights are [in, out], ``models/gpt2.py:205-251``)."""
    name: str
    transposed: bool = False
    init: Init = Init()


@dataclass(frozen=True)
class PartSpec:
    kind: str
    params: dict[str, Any] = field(default_factory=dict)
    sources: dict[str, Source] = field(default_factory=dict)


# ------------------------------------------------------------- cache needs --

@dataclass(frozen=True)
class KVNeed:
    """Keys and values in pages.  ``window`` None: every earlier key is kept;
    an integer: only the last ``window`` keys are read, earlier pages may be
    given back."""
    kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateNeed:
    """State of fixed size per request, kept in the request's slot."""
    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


# ------------------------------------------------------------------- parts --

class Part:
    """Base of every part.  Subclasses set ``KIND`` and implement ``tensors``."""

    KIND: ClassVar[str] = ""

    def tensors(self) -> dict[str, TensorDecl]:
        return {}

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        for name, tensor in tensors.items():
            setattr(self, name.replace(".", "_"), tensor)

    def cache_need(self):
        """``KVNeed``, ``StateNeed`` or None."""
        return None


class Norm(Part):
    def forward(self, x: torch.Tensor, ctx, rows: torch.Tensor | None = None) -> torch.Tensor:
        """x: residual stream [T, d] float32 -> [T or len(rows), d] compute dtype."""
        raise NotImplementedError


class Mixer(Part):
    def forward(self, h: torch.Tensor, residual: torch.Tensor, ctx, cache) -> torch.Tensor:
        """h: normed input [T, d] (compute dtype); residual: [T, d] float32.
        Returns residual + mix(h) as float32 [T, d] (it may write in place).
        ``cache`` is the ``CacheBinding`` of this run step (None if the part
        declared no need)."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, h: torch.Tensor, residual: torch.Tensor, ctx) -> torch.Tensor:
        """Returns residual + ff(h), float32 [T, d]."""
        raise NotImplementedError


class PositionEncoding(Part):
    def embedding_table(self) -> torch.Tensor | None:
        """A [positions, d] table added to the token embedding, or None."""
        return None

    def max_positions(self) -> int | None:
        return None


class Embedding(Part):
    def forward(self, ctx, position: PositionEncoding) -> torch.Tensor:
        """Residual stream [T, d] float32 of the step's tokens."""
        raise NotImplementedError


class Head(Part):
    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        """h: [S, d] normed wanted rows -> logits [S, V] float32."""
        raise NotImplementedError


class Block:
    """Arrangement of norm, mixer and feed-forward in one layer."""

    KIND: ClassVar[str] = ""

    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm, ffn: FeedForward):
        self.norm1, self.mixer, self.norm2, self.ffn = norm1, mixer, norm2, ffn

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        raise NotImplementedError


# -------------------------------------------------------------- registries --

_PARTS: dict[str, Callable[..., Part]] = {}
_BLOCKS: dict[str, type[Block]] = {}


def register_part(kind: str, factory: Callable[..., Part]) -> None:
    """``factory(**params, dtype=...)`` makes the part.  Registering a kind
    twice replaces it (tests register toy parts)."""
    _PARTS[kind] = factory


def register_block(kind: str, cls: type[Block]) -> None:
    _BLOCKS[kind] = cls


def make_part(spec: PartSpec, dtype: torch.dtype, device) -> Part:
    try:
        factory = _PARTS[spec.kind]
    except KeyError:
        raise KeyError(f"no part of kind {spec.kind!r}; registered: {sorted(_PARTS)}") from None
    return factory(**spec.params, dtype=dtype, device=device)


def make_block(kind: str, norm1, mixer, norm2, ffn) -> Block:
    try:
        cls = _BLOCKS[kind]
    except KeyError:
        raise KeyError(f"no block arrangement {kind!r}; registered: {sorted(_BLOCKS)}") from None
    return cls(norm1, mixer, norm2, ffn)


# ------------------------------------------------------------ model as data --

@dataclass(frozen=True)
class LayerSpec:
    norm1: PartSpec
    mixer: PartSpec
    norm2: PartSpec
    ffn: PartSpec
    block: str = "pre_norm"


@dataclass(frozen=True)
class RunStep:
    """One entry of the run order.  ``layer`` indexes ``ModelSpec.layers`` (a
    layer may be named twice).  ``cache_of``: index of an earlier run step whose
    cache this one reads instead of keeping its own."""
    layer: int
    cache_of: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: PartSpec
    position: PartSpec
    layers: tuple[LayerSpec, ...]
    order: tuple[RunStep, ...]
    final_norm: PartSpec
    head: PartSpec

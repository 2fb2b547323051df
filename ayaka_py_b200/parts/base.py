"""What a part is, and the registries that the model is built from.

A model is put together from parts: an embedding, a position encoding, and for
every layer a set of named parts (for GPT-2 a norm, a mixer (attention here), a
second norm and a feed-forward) that a block arranges; then a final norm and a
head.  Each part

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
    given back.  Values have the keys' head count and size unless
    ``value_heads`` / ``value_dim`` say otherwise (the pages of keys and of
    values are separate tensors)."""
    kv_heads: int
    head_dim: int
    window: int | None = None
    value_heads: int | None = None
    value_dim: int | None = None

    @property
    def v_heads(self) -> int:
        return self.kv_heads if self.value_heads is None else self.value_heads

    @property
    def v_dim(self) -> int:
        return self.head_dim if self.value_dim is None else self.value_dim

    def elements_per_token(self) -> int:
        """Key and value elements that one token takes in one layer."""
        return self.kv_heads * self.head_dim + self.v_heads * self.v_dim


@dataclass(frozen=True)
class StateNeed:
    """State of fixed size per request, kept in the request's slot."""
    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


# ------------------------------------------------------------------- parts --

class NotLowered(Exception):
    """A part cannot describe its step as operations of the native step program; the model then
    runs its steps through ``forward``."""


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

    def set_position(self, position: "PositionEncoding") -> None:
        """The model's position encoding, handed to every part of every layer when the
        model is built.  Parts that apply positions themselves (an attention that
        rotates queries and keys) keep it; the default ignores it."""

    def lower(self, builder, *args, **kwargs):
        """Optional: record what ``forward`` launches as operations of a step program
        (``engine/program.py``) and return the buffer that holds the result; the arguments
        mirror ``forward`` with buffers in the place of tensors.  The default says that
        the part cannot, which keeps its model on ``forward``."""
        raise NotLowered(type(self).__name__)


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
    # A position encoding that acts on queries and keys sets this to a method
    # ``rotate_qk(q, k, heads, kv_heads, head_dim, ctx)`` that turns the step's q and k rows
    # in place (``ctx.positions`` gives each row's position); None: nothing to do.
    rotate_qk = None

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
    """Arrangement of a layer's parts: which runs on what, in which order.

    ``PARTS`` names the parts the arrangement needs (a layer's spec must name
    exactly these); each is also reachable as an attribute.  ``forward`` gets the
    residual stream and, for the parts that declared a cache need, their
    ``CacheBinding`` by part name."""

    KIND: ClassVar[str] = ""
    PARTS: ClassVar[tuple[str, ...]] = ()

    def __init__(self, parts: dict[str, Part]):
        missing, extra = set(self.PARTS) - set(parts), set(parts) - set(self.PARTS)
        if missing or extra:
            raise ValueError(f"arrangement {self.KIND!r} takes the parts {list(self.PARTS)}: "
                             f"missing {sorted(missing)}, not used {sorted(extra)}")
        self.parts = dict(parts)
        for name, part in parts.items():
            setattr(self, name, part)

    def forward(self, x: torch.Tensor, ctx, caches: dict) -> torch.Tensor:
        raise NotImplementedError

    def lower(self, builder, x: int, caches: dict) -> int:
        """Optional, as ``Part.lower``: the arrangement over buffers."""
        raise NotLowered(type(self).__name__)


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


def make_block(kind: str, parts: dict[str, Part]) -> Block:
    try:
        cls = _BLOCKS[kind]
    except KeyError:
        raise KeyError(f"no block arrangement {kind!r}; registered: {sorted(_BLOCKS)}") from None
    return cls(parts)


# ------------------------------------------------------------ model as data --

@dataclass(frozen=True)
class LayerSpec:
    """A layer as data: its parts by name, in the order in which they are built (and in
    which their tensors are listed), and the arrangement (``register_block``) that runs
    them.  Nothing fixes how many parts a layer has or what they are called: an
    arrangement with four norms, with one norm that feeds mixer and feed-forward side
    by side, or without a feed-forward is another ``Block`` and another tuple here."""
    parts: tuple[tuple[str, PartSpec], ...]
    block: str = "pre_norm"

    def part(self, name: str) -> PartSpec:
        return dict(self.parts)[name]


def pre_norm_layer(norm1: PartSpec, mixer: PartSpec, norm2: PartSpec, ffn: PartSpec) -> LayerSpec:
    """x += mixer(norm1(x)); x += ffn(norm2(x)): the arrangement ``pre_norm``."""
    return LayerSpec((("norm1", norm1), ("mixer", mixer), ("norm2", norm2), ("ffn", ffn)), "pre_norm")


@dataclass(frozen=True)
class RunStep:
    """One entry of the run order.  ``layer`` indexes ``ModelSpec.layers`` (a
    layer may be named twice).  ``cache_of``: index of an earlier run step whose
    caches this one reads instead of keeping its own."""
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

"""Parts that models are put together from.  Importing this package registers
the built-in kinds."""

from . import attention, block, embedding, head, mlp, norm, position  # noqa: F401
from .base import (Block, Embedding, FeedForward, Head, Init, KVNeed, LayerSpec, Mixer, ModelSpec,
                   Norm, Part, PartSpec, PositionEncoding, RunStep, Source, StateNeed, TensorDecl,
                   make_block, make_part, pre_norm_layer, register_block, register_part)

__all__ = ["Part", "Norm", "Mixer", "FeedForward", "PositionEncoding", "Embedding", "Head", "Block",
           "Init", "TensorDecl", "Source", "PartSpec", "LayerSpec", "RunStep", "ModelSpec", "KVNeed",
           "StateNeed", "pre_norm_layer", "register_part", "register_block", "make_part", "make_block"]

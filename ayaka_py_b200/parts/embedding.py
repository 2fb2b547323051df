"""Token embedding, fused with a learned position table when the position
encoding offers one (``models/gpt2.py:516-517``)."""

from __future__ import annotations

import torch

from .. import ops
from .base import Embedding, TensorDecl, register_part


class TokenEmbedding(Embedding):
    KIND = "token_embedding"

    def __init__(self, vocab: int, width: int, dtype=torch.float32, device="cuda"):
        self.vocab, self.width = vocab, width
        self.weight = None

    def tensors(self):
        return {"weight": TensorDecl((self.vocab, self.width), "matrix")}

    def forward(self, ctx, position):
        return ops.embed(ctx.tokens, ctx.positions, self.weight, position.embedding_table())

    def lower(self, builder, position):
        return builder.embed(self.weight, position.embedding_table())


register_part(TokenEmbedding.KIND, TokenEmbedding)

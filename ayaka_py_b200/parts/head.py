"""Logits of the wanted rows: h @ W[:V]^T, no bias, float32 out
(``models/_common.py:248-253``, ``layers/embedding.py:741-747``)."""

from __future__ import annotations

import torch

from .. import ops
from .base import Head, TensorDecl, register_part


class LMHead(Head):
    KIND = "lm_head"

    def __init__(self, vocab: int, width: int, dtype=torch.float32, device="cuda"):
        self.vocab, self.width = vocab, width
        self.weight = None

    def tensors(self):
        return {"weight": TensorDecl((self.vocab, self.width), "matrix")}

    def forward(self, h, ctx):
        return ops.linear(h, self.weight, None, out_dtype=torch.float32)

    def lower(self, builder, h):
        from ..engine.program import LOGITS
        return builder.linear(h, self.weight, None, out_dtype=torch.float32, out=LOGITS, wanted=True)


register_part(LMHead.KIND, LMHead)

"""LayerNorm: statistics and affine in 32-bit (``layers/norm.py:198-205``)."""

from __future__ import annotations

import torch

from .. import ops
from .base import Norm, TensorDecl, register_part


class LayerNorm(Norm):
    KIND = "layernorm"

    def __init__(self, width: int, eps: float, bias: bool = True, dtype=torch.float32, device="cuda"):
        self.width, self.eps, self.has_bias = width, float(eps), bias
        self.dtype = dtype
        self.weight = None
        self.bias = None

    def tensors(self):
        out = {"weight": TensorDecl((self.width,), "vector")}
        if self.has_bias:
            out["bias"] = TensorDecl((self.width,), "vector")
        return out

    def forward(self, x, ctx, rows=None):
        return ops.layernorm(x, self.weight, self.bias, self.eps, self.dtype, rows=rows)

    def lower(self, builder, x, wanted=False):
        return builder.layernorm(x, self.weight, self.bias, self.eps, self.width, self.dtype, wanted=wanted)


register_part(LayerNorm.KIND, LayerNorm)

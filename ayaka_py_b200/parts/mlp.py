"""Dense feed-forward: up projection, activation, down projection, residual
(``models/gpt2.py:400-403``, ``:437-438``).  Bias, activation (in 32-bit) and
the residual sum are fused into the two matrix products' epilogues."""

from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, TensorDecl, register_part


class MLP(FeedForward):
    KIND = "mlp"

    def __init__(self, width: int, inner: int, activation: str, bias: bool = True,
                 dtype=torch.float32, device="cuda"):
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"unknown activation {activation!r}; known: {sorted(ops.ACTIVATIONS)}")
        self.width, self.inner, self.activation, self.has_bias = width, inner, activation, bias
        self.dtype = dtype
        self.up_weight = self.up_bias = self.down_weight = self.down_bias = None

    def tensors(self):
        out = {"up_weight": TensorDecl((self.inner, self.width), "matrix"),
               "down_weight": TensorDecl((self.width, self.inner), "matrix")}
        if self.has_bias:
            out["up_bias"] = TensorDecl((self.inner,), "vector")
            out["down_bias"] = TensorDecl((self.width,), "vector")
        return out

    def forward(self, h, residual, ctx):
        u = ops.linear(h, self.up_weight, self.up_bias, activation=self.activation, out_dtype=self.dtype)
        return ops.linear(u, self.down_weight, self.down_bias, residual=residual,
                          out_dtype=torch.float32, out=residual)

    def lower(self, builder, h, residual):
        u = builder.linear(h, self.up_weight, self.up_bias, activation=self.activation, out_dtype=self.dtype)
        out = builder.linear(u, self.down_weight, self.down_bias, residual=residual, out_dtype=torch.float32, out=residual)
        builder.release(u)
        return out


register_part(MLP.KIND, MLP)

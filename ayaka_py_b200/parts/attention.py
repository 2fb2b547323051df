"""Causal multi-head attention over the paged cache (``models/gpt2.py:364-372``).

Fused query/key/value projection (features in the order q | k | v), append of
the step's keys and values to the pages, attention of the step's rows over the
cache, output projection with the residual sum in its epilogue.  Heads, key/value
heads (grouped queries), head size, score scale and an optional window are
parameters; a run step that reads another's cache appends nothing."""

from __future__ import annotations

import torch

from .. import ops
from .base import KVNeed, Mixer, TensorDecl, register_part


class Attention(Mixer):
    KIND = "attention"

    def __init__(self, width: int, num_heads: int, head_dim: int, scale: float,
                 kv_heads: int | None = None, window: int | None = None, bias: bool = True,
                 dtype=torch.float32, device="cuda"):
        kv_heads = kv_heads or num_heads
        if num_heads % kv_heads:
            raise ValueError(f"{num_heads} heads cannot share {kv_heads} key/value heads")
        if not 1 <= head_dim <= 256:
            raise ValueError(f"head size {head_dim} is not in [1, 256]: the attention kernels keep a head's row in "
                             f"registers and shared memory sized for at most 256 elements")
        if window is not None and window < 1:
            raise ValueError("window must be positive or None")
        self.width, self.num_heads, self.kv_heads, self.head_dim = width, num_heads, kv_heads, head_dim
        self.scale, self.window, self.has_bias = float(scale), window, bias
        self.dtype = dtype
        self.q_width = num_heads * head_dim
        self.kv_width = kv_heads * head_dim
        self.qkv_weight = self.qkv_bias = self.out_weight = self.out_bias = None
        self.position = None

    def set_position(self, position) -> None:
        self.position = position

    def tensors(self):
        total = self.q_width + 2 * self.kv_width
        out = {"qkv_weight": TensorDecl((total, self.width), "matrix"),
               "out_weight": TensorDecl((self.width, self.q_width), "matrix")}
        if self.has_bias:
            out["qkv_bias"] = TensorDecl((total,), "vector")
            out["out_bias"] = TensorDecl((self.width,), "vector")
        return out

    def cache_need(self):
        return KVNeed(self.kv_heads, self.head_dim, self.window)

    def forward(self, h, residual, ctx, cache):
        kcache, vcache = ctx.cache.kv_layer(cache.group, cache.layer)
        table = ctx.tables[cache.group]
        rotate = self.position.rotate_qk if self.position is not None else None
        # Rows of prompts whose keys go into the cache as the projection makes them: the product may
        # file them itself.  (A decode step's are filed by its attention kernel, rotated keys after
        # the rotation.)
        filing = None
        if cache.writes and rotate is None and ctx.max_q_len > 1:
            filing = ops.KVAppend(kcache, vcache, ctx.row_req, ctx.positions, table, self.q_width, self.kv_width)
        qkv = ops.linear(h, self.qkv_weight, self.qkv_bias, out_dtype=self.dtype, kv=filing)
        q = qkv[:, :self.q_width]
        k = qkv[:, self.q_width:self.q_width + self.kv_width]
        v = qkv[:, self.q_width + self.kv_width:]
        if rotate is not None:
            rotate(q, k, self.num_heads, self.kv_heads, self.head_dim, ctx)
        filed = filing is not None and filing.done
        o = ops.attention(q, kcache, vcache, table, ctx, self.num_heads, self.scale, self.window,
                          append=(k, v) if cache.writes and not filed else None)
        return ops.linear(o, self.out_weight, self.out_bias, residual=residual,
                          out_dtype=torch.float32, out=residual)


    def lower(self, builder, h, residual, cache):
        from .base import NotLowered
        if self.position is not None and self.position.rotate_qk is not None:
            raise NotLowered("queries and keys are turned by the position encoding's own code")
        filing = (cache, self.q_width, self.kv_width) if cache.writes else None
        made = builder.linear(h, self.qkv_weight, self.qkv_bias, out_dtype=self.dtype, filing=filing)
        qkv, slot = made if filing is not None else (made, -1)
        o = builder.attention(qkv, cache, heads=self.num_heads, kv_heads=self.kv_heads, head_dim=self.head_dim,
                              scale=self.scale, window=self.window, dtype=self.dtype, filed_slot=slot)
        builder.release(qkv)
        out = builder.linear(o, self.out_weight, self.out_bias, residual=residual, out_dtype=torch.float32, out=residual)
        builder.release(o)
        return out


register_part(Attention.KIND, Attention)

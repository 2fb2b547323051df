"""Arrangements of a layer's parts."""

from __future__ import annotations

from .base import Block, register_block


class PreNormBlock(Block):
    """x += mixer(norm1(x)); x += ffn(norm2(x))  (``models/gpt2.py:435-438``).
    The residual stream x is float32; the sums are made in the mixer's and the
    feed-forward's last epilogue."""

    KIND = "pre_norm"
    PARTS = ("norm1", "mixer", "norm2", "ffn")

    def forward(self, x, ctx, caches):
        x = self.mixer.forward(self.norm1.forward(x, ctx), x, ctx, caches.get("mixer"))
        return self.ffn.forward(self.norm2.forward(x, ctx), x, ctx)

    def lower(self, builder, x, caches):
        h = self.norm1.lower(builder, x)
        x = self.mixer.lower(builder, h, x, caches.get("mixer"))
        builder.release(h)
        h = self.norm2.lower(builder, x)
        x = self.ffn.lower(builder, h, x)
        builder.release(h)
        return x


register_block(PreNormBlock.KIND, PreNormBlock)

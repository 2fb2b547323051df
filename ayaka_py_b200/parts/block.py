"""Arrangements of norm, mixer and feed-forward in a layer."""

from __future__ import annotations

from .base import Block, register_block


class PreNormBlock(Block):
    """x += mixer(norm1(x)); x += ffn(norm2(x))  (``models/gpt2.py:435-438``).
    The residual stream x is float32; the sums are made in the mixer's and the
    feed-forward's last epilogue."""

    KIND = "pre_norm"

    def forward(self, x, ctx, cache):
        x = self.mixer.forward(self.norm1.forward(x, ctx), x, ctx, cache)
        return self.ffn.forward(self.norm2.forward(x, ctx), x, ctx)


register_block(PreNormBlock.KIND, PreNormBlock)

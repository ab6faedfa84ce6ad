"""Block arrangements: how norms, mixer and feed-forward sit around the residual stream.

"prenorm" is the reference's layer (src/graph/llama_like.cpp:69-105):
    x = x + mixer(norm1(x));  x = x + ffn(norm2(x))
with the residual taken from the un-normed stream.
"""
from __future__ import annotations

from .base import Block, register_block


@register_block("prenorm")
class PreNormBlock(Block):
    @staticmethod
    def norm_roles():
        return ("norm1", "norm2")

    def forward(self, stream, ctx, cache, writes):
        # the outputs only go into the residual stream, so they may stay unreduced (see
        # Mixer.forward_deferred): the next norm adds the slices while it reads the row anyway
        h = self.norms["norm1"].forward(stream)
        stream.add(self.mixer.forward_deferred(h, ctx, cache, writes))
        h = self.norms["norm2"].forward(stream)
        stream.add(self.ffn.forward_deferred(h, ctx))

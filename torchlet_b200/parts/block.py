"""Arrangements of a layer's parts around the residual stream.

"pre_norm": h = x + mixer(norm(x)); x' = h + feed_forward(norm(h))
(v10_triton_paged_gqa/layer/transformer_block.py:37-40).  The stream ``acc`` is
float32; mixer and feed-forward add into it.
"""
from __future__ import annotations

from .base import BLOCKS, Block


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    norm_roles = ("mixer_norm", "feed_forward_norm")

    def forward(self, ctx, acc, cache) -> None:
        x = self.norms["mixer_norm"].apply(ctx, acc)
        self.mixer.forward(ctx, x, acc, cache)
        x = self.norms["feed_forward_norm"].apply(ctx, acc)
        self.feed_forward.forward(ctx, x, acc)

"""Rotary position encoding, split-half pairing (element i with i + d/2):
y1 = x1 cos - x2 sin, y2 = x2 cos + x1 sin, angle = position * theta^(-2i/d),
angles and rotation in float32 (v10_triton_paged_gqa/layer/rope.py:18-69,
kernel/rope.py:21-41).

This encoding writes the k and v heads to the cache pages of each token in the same pass
(``stores_kv``): the encoded key never needs to exist anywhere else.
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.spec import PartSpec
from .base import POSITIONS, Positions


@POSITIONS.register("rotary_split_half")
class RotarySplitHalf(Positions):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.head_dim = int(spec.params["head_dim"])
        self.theta = float(spec.params["theta"])
        if self.head_dim % 2:
            raise ValueError("head_dim must be even for split-half rotation")
        self.inv_freq = None

    def load(self, tensors: dict, prefix: str, device, dtype) -> None:
        # exactly the reference's table: 1 / theta ** (arange(0, d, 2) / d) in float32
        i = torch.arange(0, self.head_dim, 2, dtype=torch.float32)
        self.inv_freq = (1.0 / (self.theta ** (i / self.head_dim))).to(device)

    accepts_partials = True
    stores_kv = True

    def encode_and_store(self, ctx, qkv, num_heads, num_kv_heads, cache, partials=None) -> None:
        """``partials``: (float32 split sums, splits, bias) of the qkv product when the
        mixer left it unfinished; the sum, the bias, the rotation and the store then run as
        one kernel and ``qkv`` receives the encoded q."""
        if partials is not None:
            ops.finish_qkv_rope(partials[0], partials[1], partials[2], qkv, ctx.positions, ctx.token_req,
                                cache.block_table, cache.pages, self.inv_freq, num_heads, num_kv_heads,
                                self.head_dim, cache.page_size, write_kv=cache.writable)
            return
        ops.rope_kv(qkv, ctx.positions, ctx.token_req, cache.block_table, cache.pages, self.inv_freq,
                    num_heads, num_kv_heads, self.head_dim, cache.page_size, write_kv=cache.writable)

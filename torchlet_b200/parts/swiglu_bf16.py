"""Choice of the fused bfloat16 tensor-core feed-forward kernels.  Returns False when
none takes the sizes; the caller then uses the any-size kernels."""
from __future__ import annotations


def forward(ffn, ctx, x, acc) -> bool:
    return False

"""Choice of the bfloat16 tensor-core matrix-product kernel for a ``Linear``.

Returns False when no tensor-core kernel takes the sizes; the caller then uses the
CUDA-core kernel, which takes every size.
"""
from __future__ import annotations


def forward(linear, x, out, accumulate: bool) -> bool:
    return False

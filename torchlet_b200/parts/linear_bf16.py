"""Choice of the bfloat16 tensor-core matrix-product kernel for a ``Linear``.

Returns False when the tcgen05 kernel does not take the sizes (K or a row stride not a
multiple of 8 elements); the caller then uses the CUDA-core kernel, which takes every size.
"""
from __future__ import annotations

import torch

from .. import ops


def forward(linear, x, out, accumulate: bool) -> bool:
    if not ops.gemm_tc_supported(x, linear.weight):
        return False
    if accumulate:
        epilogue = ops.EPI_ACCUM_F32
    elif out.dtype == torch.bfloat16:
        epilogue = ops.EPI_STORE_BF16
    else:
        epilogue = ops.EPI_STORE_F32
    ops.gemm_tc(x, linear.weight, out, linear.bias, epilogue)
    return True

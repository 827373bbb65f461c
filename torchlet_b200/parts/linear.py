"""A weight matrix [out, in] with its matrix product, y = x W^T + b
(nn.Linear layout as in the reference, v10_triton_paged_gqa/layer/gqa.py:40-45).

The matrix is held in the compute dtype, the bias in float32.  ``forward`` picks the
kernel: the CUDA-core kernel for float32 (the true 32-bit path) and for any size the
tensor-core kernels refuse; tcgen05 kernels for bfloat16 otherwise.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops


class Linear:
    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor], device, dtype: torch.dtype):
        self.out_features, self.in_features = weight.shape
        self.weight = weight.to(device=device, dtype=dtype).contiguous()
        self.bias = None if bias is None else bias.to(device=device, dtype=torch.float32).contiguous()
        self.dtype = dtype

    @classmethod
    def from_device_weight(cls, weight: torch.Tensor) -> "Linear":
        """Share an already resident matrix (tied embedding and LM head)."""
        self = cls.__new__(cls)
        self.out_features, self.in_features = weight.shape
        self.weight, self.bias, self.dtype = weight, None, weight.dtype
        return self

    def deferred(self, ctx, x: torch.Tensor):
        """For few tokens in bfloat16: run the product but leave its split partial sums
        for a fused finishing kernel.  Returns (partials, splits) or None (not applicable;
        use ``forward``)."""
        if self.dtype != torch.bfloat16 or not ops.gemm_tc_supported(x, self.weight):
            return None
        return ops.gemm_tc_deferred(x, self.weight)

    def accumulate_later(self, ctx, x: torch.Tensor, acc: torch.Tensor) -> bool:
        """acc += x W^T + b, with the final sum left to whoever reads ``acc`` next
        (``ctx.leave_pending``: the next norm, or ``ctx.flush_pending``).
        False: not applicable, nothing was done."""
        result = self.deferred(ctx, x)
        if result is None:
            return False
        ctx.leave_pending(result[0], result[1], self.bias, acc)
        return True

    def forward(self, x: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
        """out (+)= x W^T + b.  ``accumulate`` needs a float32 ``out`` (the residual stream)."""
        if self.dtype == torch.bfloat16:
            from . import linear_bf16

            if linear_bf16.forward(self, x, out, accumulate):
                return
        ops.gemm_simt(x, self.weight, out, self.bias, accumulate)

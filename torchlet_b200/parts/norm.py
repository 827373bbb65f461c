"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, float32 inside
(v10_triton_paged_gqa/layer/rms_norm.py:7-25, kernel/rms_norm.py:13-22)."""
from __future__ import annotations

import torch

from .. import ops
from ..config.spec import PartSpec
from .base import NORMS, Norm, TensorSpec


@NORMS.register("rms_norm")
class RMSNorm(Norm):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.weight = None

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        return [TensorSpec(prefix + "weight", (int(spec.params["size"]),), init="ones")]

    def load(self, tensors: dict, prefix: str, device, dtype) -> None:
        self.weight = tensors[prefix + "weight"].to(device=device, dtype=torch.float32).contiguous()

    fuses_pending = True  # a product's unfinished sum into the stream is completed in the norm's own kernel

    def forward(self, ctx, acc, out=None, rows=None, name="normed"):
        """Normed rows of the float32 stream ``acc`` in the compute dtype; ``rows``
        (int32) selects and orders the rows, default all."""
        count = acc.shape[0] if rows is None else rows.numel()
        if out is None:
            out = ctx.buffer(name, (count, self.size), ctx.dtype)
        if rows is None and out.dtype == torch.bfloat16:
            pending = ctx.take_pending(acc)
            if pending is not None:  # finish the sum and norm in one kernel
                ops.finish_accum_norm(pending.partials, pending.splits, pending.bias, acc, self.weight, self.eps, out)
                return out
        ctx.flush_pending()
        ops.rms_norm(acc, self.weight, self.eps, out, rows)
        return out

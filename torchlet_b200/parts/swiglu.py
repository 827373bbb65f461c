"""SwiGLU feed-forward: down(silu(gate(x)) * up(x)), no biases, activation in float32
(v10_triton_paged_gqa/layer/ffn_swiglu.py:7-60, kernel/ffn_swiglu.py:139-164;
formula v08_paged_gqa_py/layer/ffn_swiglu.py:12-15)."""
from __future__ import annotations

import torch

from .. import ops
from ..config.spec import PartSpec
from .base import FEED_FORWARDS, FeedForward, TensorSpec
from .linear import Linear


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.hidden_size = int(spec.params["hidden_size"])
        self.intermediate_size = int(spec.params["intermediate_size"])
        self.gate_up_proj: Linear | None = None
        self.gate_up_interleaved = None  # bfloat16 fused path: gate/up rows interleaved by 16
        self.down_proj: Linear | None = None

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        hidden, inter = int(spec.params["hidden_size"]), int(spec.params["intermediate_size"])
        return [
            TensorSpec(prefix + "gate_proj.weight", (inter, hidden)),
            TensorSpec(prefix + "up_proj.weight", (inter, hidden)),
            TensorSpec(prefix + "down_proj.weight", (hidden, inter)),
        ]

    def load(self, tensors: dict, prefix: str, device, dtype) -> None:
        from . import swiglu_bf16

        gate, up = tensors[prefix + "gate_proj.weight"], tensors[prefix + "up_proj.weight"]
        if dtype == torch.bfloat16 and swiglu_bf16.usable(self.hidden_size, self.intermediate_size):
            self.gate_up_interleaved = swiglu_bf16.interleave(
                gate.to(device=device, dtype=dtype), up.to(device=device, dtype=dtype))
        else:
            self.gate_up_proj = Linear(torch.cat([gate, up], dim=0), None, device, dtype)
        self.down_proj = Linear(tensors[prefix + "down_proj.weight"], None, device, dtype)

    def forward(self, ctx, x, acc) -> None:
        tokens = x.shape[0]
        from . import swiglu_bf16

        if ctx.dtype == torch.bfloat16 and swiglu_bf16.forward(self, ctx, x, acc):
            return
        gate_up = ctx.buffer("swiglu.gate_up", (tokens, 2 * self.intermediate_size), ctx.dtype)
        self.gate_up_proj.forward(x, gate_up)
        act = ctx.buffer("swiglu.act", (tokens, self.intermediate_size), ctx.dtype)
        ops.swiglu(gate_up, act)
        self.down_proj.forward(act, acc, accumulate=True)

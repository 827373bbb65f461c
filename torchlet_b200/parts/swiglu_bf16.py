"""The fused bfloat16 feed-forward: gate and up projections as ONE tcgen05 product whose
epilogue applies silu(gate) * up, so the [T, 2I] intermediate never reaches memory.

For that the rows of the gate and up matrices are interleaved in blocks of 16
(g0..g15, u0..u15, g16..g31, u16..u31, ...): a 32-column chunk of the accumulator then
holds 16 gate values and their 16 up values.  Needs intermediate_size % 16 == 0 and
hidden_size % 8 == 0; otherwise the feed-forward uses the separate kernels.
"""
from __future__ import annotations

import torch

from .. import ops

BLOCK = 16


def usable(hidden_size: int, intermediate_size: int) -> bool:
    return intermediate_size % BLOCK == 0 and hidden_size % 8 == 0


def interleave(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    inter, hidden = gate.shape
    g = gate.view(inter // BLOCK, BLOCK, hidden)
    u = up.view(inter // BLOCK, BLOCK, hidden)
    return torch.cat([g, u], dim=1).reshape(2 * inter, hidden).contiguous()


def forward(ffn, ctx, x, acc) -> bool:
    if ffn.gate_up_interleaved is None:
        return False
    tokens = x.shape[0]
    act = ctx.buffer("swiglu.act", (tokens, ffn.intermediate_size), torch.bfloat16)
    ops.gemm_tc(x, ffn.gate_up_interleaved, act, None, ops.EPI_SWIGLU_BF16)
    if not ffn.down_proj.accumulate_later(ctx, act, acc):
        ffn.down_proj.forward(act, acc, accumulate=True)
    return True
